"""`tbik_gemm_static`: the GEMM entry point for callers that cannot allocate device memory.

Some hosts of this library have no device allocator to offer (a C / Go / Rust service binding the
C ABI directly) or must not call one at the point of use (an inference server that has handed every
free byte of HBM to its KV cache).  For them the library carries its own fixed scratch array.  This
test calls the entry point through the C ABI twice in a row, on different operands, and requires
the result to equal -- bit for bit, the tolerance of every other integer-exactness test here --
what `tbik_gemm_ws` returns with a caller-owned scratch buffer, and on integer-valued operands what
the CPU oracle returns.  It also checks that the call leaves the device's free memory unchanged, that a
size no schedule of which fits the built-in array is refused before anything is launched, and (with a
second GPU) that each device gets its own array.
The file name sorts last so that a failure here cannot hide the other tests in a `-x` run.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _bits(t):
    return t.contiguous().view(torch.int16)


def _run(fn, A, W, extra=()):
    from llm_reproducibility_b200 import _lib
    M, K = A.shape
    N = W.shape[0]
    C = torch.empty(M, N, dtype=A.dtype, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    rc = fn(A.data_ptr(), W.data_ptr(), C.data_ptr(), M, N, K, K, K, N, _lib.DTYPE_BF16, 256, _lib.NODE_INPUT, *extra, s)
    assert rc == 0, _lib.last_error()
    torch.cuda.synchronize()
    return C


@pytest.mark.parametrize("M,K,N", [
    (64, 12288, 4096),     # decode-sized: K-slabs, the slab roots live in the scratch
    (300, 65536, 1024),    # 8-level tree: one stack level beyond tensor memory and shared memory goes to scratch
    (16, 12288, 1000),     # K-slabs with N not a multiple of 8 columns: padded rows of roots, scalar stores of C
])
def test_static_scratch_entry_point_matches_workspace_entry_point_twice(M, K, N):
    from llm_reproducibility_b200 import _lib
    L = _lib.lib()
    need = L.tbik_gemm_workspace_bytes(M, N, K, 256)
    assert 0 < need <= L.tbik_gemm_static_scratch_bytes() and L.tbik_gemm_static_accepts(M, N, K, 256) == 1
    ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
    g = torch.Generator(device="cuda").manual_seed(2024)
    for call in range(2):                  # second call: new operands, scratch still holds the first call's words
        A = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
        W = (torch.randn(N, K, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
        want = _run(L.tbik_gemm_ws, A, W, extra=(ws.data_ptr(), ws.numel()))
        free_before = torch.cuda.mem_get_info()[0]
        got = _run(L.tbik_gemm_static, A, W)
        assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the device's free memory"
        assert torch.equal(_bits(got), _bits(want)), f"call {call}"
    st = (ctypes.c_uint32 * 4)()
    assert L.tbik_gemm_status(st) == 0 and st[0] == 0


def test_static_scratch_entry_point_matches_the_oracle_twice():
    """Integer-valued operands: every leaf sum is exact, so the CPU restatement of the reference's tree must be
    reproduced bit for bit -- on two calls in a row that share the built-in array (K-slabs: roots and counters)."""
    from llm_reproducibility_b200 import _lib
    from oracle.tbik_ref import exact_int_inputs, tbik_matmul_ref
    L = _lib.lib()
    for call, (M, K, N) in enumerate(((16, 12288, 520), (16, 4096, 1000))):
        A, B = exact_int_inputs(M, K, N, torch.bfloat16, seed=31 + call, amax=7)
        got = _run(L.tbik_gemm_static, A.cuda(), B.cuda().t().contiguous())
        assert torch.equal(_bits(got.cpu()), _bits(tbik_matmul_ref(A, B))), f"call {call}"


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs a second GPU")
def test_static_scratch_entry_point_on_a_second_device():
    """The array's address is looked up per device: the same call on cuda:1 must use cuda:1's copy."""
    from llm_reproducibility_b200 import _lib
    L = _lib.lib()
    M, K, N = 64, 12288, 4096
    outs = []
    for dev in (0, 1):
        with torch.cuda.device(dev):
            g = torch.Generator(device=f"cuda:{dev}").manual_seed(99)
            A = torch.randn(M, K, generator=g, device=f"cuda:{dev}").to(torch.bfloat16)
            W = (torch.randn(N, K, generator=g, device=f"cuda:{dev}") * 0.02).to(torch.bfloat16)
            C = torch.empty(M, N, dtype=A.dtype, device=f"cuda:{dev}")
            rc = L.tbik_gemm_static(A.data_ptr(), W.data_ptr(), C.data_ptr(), M, N, K, K, K, N, _lib.DTYPE_BF16, 256,
                                    _lib.NODE_INPUT, torch.cuda.current_stream().cuda_stream)
            assert rc == 0, _lib.last_error()
            torch.cuda.synchronize()
            outs.append(C.cpu())
    assert torch.equal(_bits(outs[0]), _bits(outs[1]))


def test_static_scratch_entry_point_refuses_sizes_beyond_its_array():
    from llm_reproducibility_b200 import _lib
    L = _lib.lib()
    M, K, N = 8192, 1 << 23, 4096         # 15-level tree: 8 stack levels x 32 KiB x 148 CTAs > 32 MiB
    assert L.tbik_gemm_workspace_bytes(M, N, K, 256) > L.tbik_gemm_static_scratch_bytes()
    assert L.tbik_gemm_static_accepts(M, N, K, 256) == 0     # asked first: the call below must not reach a launch
    assert L.tbik_gemm_static_accepts(64, 4096, 12288, 256) == 1
    x = torch.zeros(4096, dtype=torch.bfloat16, device="cuda")   # never dereferenced: the call is refused first
    rc = L.tbik_gemm_static(x.data_ptr(), x.data_ptr(), x.data_ptr(), M, N, K, K, K, N, _lib.DTYPE_BF16, 256,
                            _lib.NODE_INPUT, torch.cuda.current_stream().cuda_stream)
    assert rc == -2
    msg = _lib.last_error()
    assert "built into the library" in msg and "tbik_gemm_ws" in msg
    torch.cuda.synchronize()
