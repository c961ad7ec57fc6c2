"""End-to-end check under vLLM: greedy tokens and logprobs must not depend on the tensor-parallel degree or on
the batch size (counterpart of the reference's simple_inference.py:62-194, which compares three engines:
tp=1/bs=4, tp=4/bs=4, tp=4/bs=2).

    python -m llm_reproducibility_b200.simple_inference [--tps 1,2] [--batch-sizes 4,2] [--tokens 32] [--graphs]

No checkpoint is downloaded: a small Qwen3-shaped model (random weights, fixed seed) is written to a scratch
folder with `transformers`, and every engine loads that same folder, so the shards of a TP = n engine are slices
of the TP = 1 weights.  Prompts are fixed pseudo-random token ids (no tokenizer).  Each engine runs in a process of
its own (GPU memory is returned in between) with VLLM_BATCH_INVARIANT=1 (vLLM's own batch-invariant kernels for
everything that is not row-split) and VLLM_TP_INVARIANT=1 (`apply_patches()` swaps RowParallelLinear.forward for
the tree matmul + tree all-reduce of this package).  `--graphs` runs with CUDA graphs (enforce_eager=False), which
exercises `CustomTreeAllreduce.capture()` and the registered buffer under capture.
Exit code 0 = every engine produced the same tokens and the same logprobs, bit for bit.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

MODEL = dict(hidden_size=1024, intermediate_size=3072, num_hidden_layers=4, num_attention_heads=8,
             num_key_value_heads=4, head_dim=128, vocab_size=8192, max_position_embeddings=2048,
             rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=False)


def write_model(path: str, seed: int = 0) -> None:
    import torch
    from transformers import Qwen3Config, Qwen3ForCausalLM
    torch.manual_seed(seed)
    cfg = Qwen3Config(**MODEL)
    model = Qwen3ForCausalLM(cfg).to(torch.bfloat16)
    model.save_pretrained(path, safe_serialization=True)


def write_plugin(path: str) -> None:
    """A minimal installed-package record that registers `apply_patches` as a vLLM general plugin.

    vLLM starts its tensor-parallel workers as fresh processes (spawn), so a monkey patch applied in the launching
    process never reaches them; what every vLLM process does at start-up is load the entry points of the group
    `vllm.general_plugins`.  An installed copy of this package carries that entry point in its metadata
    (pyproject.toml); for a run from a source tree the same record is written to a scratch folder that is put on
    PYTHONPATH."""
    info = os.path.join(path, "llm_reproducibility_b200_vllm_plugin-1.0.dist-info")
    os.makedirs(info, exist_ok=True)
    with open(os.path.join(info, "METADATA"), "w") as f:
        f.write("Metadata-Version: 2.1\nName: llm-reproducibility-b200-vllm-plugin\nVersion: 1.0\n")
    with open(os.path.join(info, "entry_points.txt"), "w") as f:
        f.write("[vllm.general_plugins]\ntbik_tp_invariant = llm_reproducibility_b200.patch:apply_patches\n")


def prompts(batch: int, length: int = 48):
    import random
    rng = random.Random(1234)
    return [[rng.randrange(10, MODEL["vocab_size"] - 10) for _ in range(length)] for _ in range(batch)]


def worker(args) -> None:
    os.environ.setdefault("VLLM_BATCH_INVARIANT", "1")
    os.environ.setdefault("VLLM_TP_INVARIANT", "1")
    os.environ.setdefault("VLLM_ENABLE_V1_MULTIPROCESSING", "0")
    os.environ.setdefault("VLLM_LOGGING_LEVEL", "INFO")
    import logging
    logging.basicConfig(level=logging.INFO)
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    from llm_reproducibility_b200.patch import apply_patches
    apply_patches()  # this process; the spawned workers get it through the plugin entry point (PYTHONPATH)
    from vllm import LLM, SamplingParams
    extra = {}
    if args.graphs:
        # whole-forward CUDA graphs for the decode steps, no compiler in between: the patched layer is captured
        # as it is (GEMM into the registered buffer, tree all-reduce kernel) and replayed
        extra["compilation_config"] = {"mode": 0, "cudagraph_mode": "FULL_DECODE_ONLY", "cudagraph_capture_sizes": [1, 2, 4, 8]}
    llm = LLM(model=args.model, tensor_parallel_size=args.tp, dtype="bfloat16", skip_tokenizer_init=True,
              enforce_eager=not args.graphs, max_model_len=512, gpu_memory_utilization=0.30, seed=0,
              enable_prefix_caching=False, max_num_seqs=max(8, args.bs), **extra)
    sp = SamplingParams(temperature=0.0, max_tokens=args.tokens, logprobs=0, detokenize=False, ignore_eos=True)
    all_prompts = prompts(4)
    outs = []
    for i in range(0, len(all_prompts), args.bs):  # the same four prompts, `bs` at a time
        batch = [{"prompt_token_ids": p} for p in all_prompts[i:i + args.bs]]
        for o in llm.generate(batch, sp, use_tqdm=False):
            c = o.outputs[0]
            lps = [float(step[tok].logprob) for step, tok in zip(c.logprobs, c.token_ids)]
            outs.append({"tokens": list(c.token_ids), "logprobs": lps})
    calls = sys.modules["llm_reproducibility_b200.patch.patch_tp_invariant"].CALLS
    with open(args.out, "w") as f:
        json.dump({"sequences": outs, "patched_forward_calls_in_driver_process": calls}, f)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tps", default="1,2")
    ap.add_argument("--batch-sizes", default="4,2")
    ap.add_argument("--tokens", type=int, default=32)
    ap.add_argument("--graphs", action="store_true")
    ap.add_argument("--log-dir", default="", help="keep every engine's output there")
    ap.add_argument("--worker", action="store_true")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--bs", type=int, default=4)
    ap.add_argument("--model", default="")
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    if args.worker:
        worker(args)
        return 0
    tmp = tempfile.mkdtemp(prefix="tbik_e2e_")
    model_dir = os.path.join(tmp, "model")
    write_model(model_dir)
    plugin_dir = os.path.join(tmp, "plugin")
    write_plugin(plugin_dir)
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([plugin_dir, ROOT] + ([env["PYTHONPATH"]] if env.get("PYTHONPATH") else []))
    env.setdefault("VLLM_BATCH_INVARIANT", "1")
    env.setdefault("VLLM_TP_INVARIANT", "1")
    results = {}
    for tp in [int(x) for x in args.tps.split(",")]:
        for bs in [int(x) for x in args.batch_sizes.split(",")]:
            out = os.path.join(tmp, f"tp{tp}_bs{bs}.json")
            cmd = [sys.executable, "-m", "llm_reproducibility_b200.simple_inference", "--worker", "--tp", str(tp), "--bs", str(bs),
                   "--tokens", str(args.tokens), "--model", model_dir, "--out", out] + (["--graphs"] if args.graphs else [])
            proc = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=1200, env=env)
            if args.log_dir:
                with open(os.path.join(args.log_dir, f"engine_tp{tp}_bs{bs}.log"), "w") as f:
                    f.write(proc.stdout + "\n---- stderr ----\n" + proc.stderr)
            if proc.returncode != 0 or not os.path.isfile(out):
                print(f"engine tp={tp} bs={bs} failed (rc {proc.returncode}):\n{proc.stdout[-2000:]}\n{proc.stderr[-4000:]}")
                return 2
            with open(out) as f:
                payload = json.load(f)
            results[(tp, bs)] = payload["sequences"]
            print(f"engine tp={tp} bs={bs}: {len(results[(tp, bs)])} sequences, first tokens {results[(tp, bs)][0]['tokens'][:8]}, "
                  f"patched forwards seen by the driver process: {payload['patched_forward_calls_in_driver_process']}")
    keys = sorted(results)
    base = results[keys[0]]
    ok = True
    for k in keys[1:]:
        same_tok = all(a["tokens"] == b["tokens"] for a, b in zip(base, results[k]))
        max_dlp = max(abs(x - y) for a, b in zip(base, results[k]) for x, y in zip(a["logprobs"], b["logprobs"]))
        print(f"tp={keys[0][0]} bs={keys[0][1]} vs tp={k[0]} bs={k[1]}: tokens identical {same_tok}, max |delta logprob| {max_dlp}")
        ok = ok and same_tok and max_dlp == 0.0
    print("TP- and batch-invariant under vLLM" if ok else "MISMATCH")
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
