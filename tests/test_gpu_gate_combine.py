"""Gated sum of the three branch outputs: CUDA kernels (through the C interface) against the fp32 oracle, forward and
backward, contiguous and strided inputs, bf16 and fp16, head_dim 64 and 128, and a row count that is not a multiple of
the rows a warp holds."""
import pytest
import torch

from oracle import nsa_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    import native_sparse_attention_triton_b200 as pkg
    assert torch.cuda.is_available()
    return pkg.ops


def make(n, h, d, dtype, seed, strided):
    g = torch.Generator(device="cuda").manual_seed(seed)
    dev = torch.device("cuda")
    gate = torch.sigmoid(torch.randn(n, h * 3, generator=g, device=dev)).to(dtype).view(n, h, 3)
    if strided:  # head slices of wider tensors, as a caller that packs the branches side by side would pass
        wide = torch.randn(n, 3 * h, d, generator=g, device=dev).to(dtype)
        outs = [wide[:, i * h:(i + 1) * h] for i in range(3)]
    else:
        outs = [torch.randn(n, h, d, generator=g, device=dev).to(dtype) for _ in range(3)]
    dout = torch.randn(n, h, d, generator=g, device=dev).to(dtype)
    return gate, outs, dout


@pytest.mark.parametrize("n,h,d,dtype,strided", [
    (1024, 16, 128, torch.bfloat16, False),
    (777, 5, 128, torch.bfloat16, True),
    (333, 3, 64, torch.float16, False),
    (1, 1, 64, torch.bfloat16, False),
    (4096, 64, 128, torch.float16, True),
])
def test_gate_combine_matches_oracle(ops, n, h, d, dtype, strided):
    import native_sparse_attention_triton_b200 as pkg
    gate, outs, dout = make(n, h, d, dtype, 11 + n, strided)
    gate_g = gate.clone().requires_grad_(True)
    outs_g = [o.clone().requires_grad_(True) if not strided else o.detach().requires_grad_(True) for o in outs]
    y = ops.gate_combine(gate_g, *outs_g)
    assert y.is_contiguous() and y.shape == (n, h, d)
    y.backward(dout)
    # oracle: the layer's expression in fp32 on the CPU, gradients by autograd
    gate_c = gate.float().cpu().requires_grad_(True)
    outs_c = [o.float().cpu().requires_grad_(True) for o in outs]
    y_ref = O.gate_combine(gate_c, *outs_c)
    y_ref.backward(dout.float().cpu())
    tol = 1e-2  # the tolerance of the reference's own comparisons (atol = rtol = 1e-2)
    def close(a, b):
        a, b = a.detach().float().cpu(), b.detach().float()
        return float(((a - b).abs() / b.abs().clamp(min=1.0)).max()) <= tol
    assert close(y, y_ref)
    for a, b in zip(outs_g, outs_c):
        assert close(a.grad, b.grad)
    # d_gate sums head_dim products: compare relative to the magnitude of such a sum
    dg, dg_ref = gate_g.grad.float().cpu(), gate_c.grad
    assert float((dg - dg_ref).abs().max()) <= tol * max(1.0, float(dg_ref.abs().max()))
    assert pkg.device_status() == 0


def test_gate_combine_rejects_bad_arguments(ops):
    gate, outs, _ = make(8, 2, 128, torch.bfloat16, 3, False)
    with pytest.raises(AssertionError):
        ops.gate_combine(gate.float(), *outs)
    with pytest.raises(AssertionError):
        ops.gate_combine(gate[:, :, :2], *outs)
    with pytest.raises(AssertionError):
        ops.gate_combine(gate, outs[0], outs[1], outs[2][:, :1])
