"""Greedy decoding through a Qwen3-shaped decoder gives the same tokens and the same logits, bit for bit, for every
tensor-parallel degree and every batch size (the reference's end-to-end claim, simple_inference.py:133-194 and
README.md "tensor-parallel and batch invariance")."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _prompts(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    lens = [17, 9, 24, 5, 13, 21, 3, 11][:n]
    return [torch.randint(0, cfg.vocab, (L,), generator=g) for L in lens]


@pytest.fixture(scope="module")
def small_model():
    from decoder_harness import Config, Weights
    cfg = Config()
    return cfg, Weights(cfg, seed=1234)


def test_tp_and_batch_invariant_greedy_decode(small_model):
    from decoder_harness import Decoder
    cfg, w = small_model
    prompts = _prompts(cfg, 8, seed=7)
    steps = 6
    ref_ids, ref_logits = Decoder(cfg, w, tp=1).greedy(prompts, steps)
    assert ref_ids.shape == (8, steps)
    for tp in (2, 4, 8):
        ids, logits = Decoder(cfg, w, tp=tp).greedy(prompts, steps)
        assert torch.equal(ids, ref_ids), f"tp={tp}: tokens differ"
        assert torch.equal(logits.view(torch.int16), ref_logits.view(torch.int16)), f"tp={tp}: logits differ"
    # batch invariance: every sequence decoded alone, and in a batch of three, under different tp
    for b, tp in ((0, 1), (1, 2), (2, 8), (3, 4)):
        ids, logits = Decoder(cfg, w, tp=tp).greedy([prompts[b]], steps)
        assert torch.equal(ids[0], ref_ids[b]), f"sequence {b} alone at tp={tp}: tokens differ"
        assert torch.equal(logits[:, 0].view(torch.int16), ref_logits[:, b].view(torch.int16))
    ids, logits = Decoder(cfg, w, tp=4).greedy(prompts[2:5], steps)
    assert torch.equal(ids, ref_ids[2:5])
    assert torch.equal(logits.view(torch.int16), ref_logits[:, 2:5].view(torch.int16))


def test_without_tree_order_tp_changes_bits(small_model):
    """The check above is not vacuous: summing the K-shards' partials of a plain fp32-accumulated GEMM gives other bits."""
    cfg, w = small_model
    x = (torch.randn(64, cfg.intermediate, device="cuda") * 0.5).to(torch.bfloat16)
    W = w.layers[0]["wd"]
    full = (x.float() @ W.float().t()).to(torch.bfloat16)
    ks = cfg.intermediate // 4
    parts = [(x[:, r * ks:(r + 1) * ks].float() @ W[:, r * ks:(r + 1) * ks].float().t()).to(torch.bfloat16) for r in range(4)]
    split = (parts[0] + parts[1]) + (parts[2] + parts[3])
    assert not torch.equal(full, split)


def test_qwen3_8b_layer_shape_one_step():
    """Qwen3-8B's true layer shape (o_proj K=4096, down_proj K=12288), two layers, prefill and two decode steps."""
    from decoder_harness import Decoder, Weights, qwen3_8b_shape
    cfg = qwen3_8b_shape(layers=2, vocab=4096)
    w = Weights(cfg, seed=99)
    prompts = _prompts(cfg, 4, seed=3)
    ref_ids, ref_logits = Decoder(cfg, w, tp=1).greedy(prompts, 3)
    for tp in (2, 4, 8):
        ids, logits = Decoder(cfg, w, tp=tp).greedy(prompts, 3)
        assert torch.equal(ids, ref_ids), f"tp={tp}"
        assert torch.equal(logits.view(torch.int16), ref_logits.view(torch.int16)), f"tp={tp}"
    ids, logits = Decoder(cfg, w, tp=2).greedy([prompts[1]], 3)
    assert torch.equal(ids[0], ref_ids[1])
    assert torch.equal(logits[:, 0].view(torch.int16), ref_logits[:, 1].view(torch.int16))
