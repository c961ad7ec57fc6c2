"""Backward of the tree matmul (training-side counterpart of src/patch/patch_batch_invariant.py:38-73).

Gradients are held against an fp32 torch reference of the same op within a bf16 tolerance, must be bitwise
reproducible run after run, and dA must be batch-invariant (row i of dA depends on row i of dC only)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def bits(t):
    return t.contiguous().view(torch.int16)


def make(M, K, N, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    A = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16).requires_grad_(True)
    W = (torch.randn(N, K, generator=g, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_(True)
    dC = torch.randn(M, N, generator=g, device="cuda").to(torch.bfloat16)
    return A, W, dC


@pytest.mark.parametrize("M,K,N", [(300, 1024, 512), (512, 4096, 1024), (77, 768, 256)])
def test_gradients_match_fp32_reference_and_are_reproducible(M, K, N):
    from llm_reproducibility_b200.tbik.autograd import tree_linear
    A, W, dC = make(M, K, N, M + K)
    y = tree_linear(A, W)
    y.backward(dC)
    dA, dW = A.grad.clone(), W.grad.clone()
    # fp32 reference of the same op
    Af, Wf = A.detach().float().requires_grad_(True), W.detach().float().requires_grad_(True)
    (Af @ Wf.t()).backward(dC.float())
    for got, want in ((dA, Af.grad), (dW, Wf.grad)):
        err = (got.float() - want).abs().max() / want.abs().max()
        assert err.item() < 2.0e-2, err.item()
    # run again: the same bits
    A.grad = W.grad = None
    tree_linear(A, W).backward(dC)
    assert torch.equal(bits(A.grad), bits(dA)) and torch.equal(bits(W.grad), bits(dW))


def test_input_gradient_is_batch_invariant():
    from llm_reproducibility_b200.tbik.autograd import tree_matmul
    A, W, dC = make(256, 2048, 512, 3)
    tree_matmul(A, W.t()).backward(dC)
    full = A.grad.clone()
    A2 = A.detach()[:19].clone().requires_grad_(True)
    tree_matmul(A2, W.detach().t()).backward(dC[:19])
    assert torch.equal(bits(A2.grad), bits(full[:19]))
