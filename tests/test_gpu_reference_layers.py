"""The reference's own layers, unchanged, on this package's operators (BASELINE configurations 4 and 5 at reduced size).

``module.NativeSparseAttention`` (module/native_sparse_attention.py:145-238) and ``model.ToyNSALlama``
(model/toy_nsa_llama.py:206-277) are imported from ``baseline/_ref`` (skipped where it is absent) and run twice in one
process on identical weights and inputs: first bound to the reference's Triton operators, flash_attn and its own KV cache,
then -- after ``shim.install()``, ``install_sliding_window()`` and ``install_inference()`` -- bound to libnsa_b200.so.
"""
import os

import pytest
import torch

from tests import refbox

pytestmark = pytest.mark.gpu


@pytest.fixture()
def ref():
    r = refbox.load(layers=True)
    yield r
    refbox.unload()


def use_this_package():
    from native_sparse_attention_triton_b200 import shim
    shim.install(patch_loaded=True)
    assert shim.install_sliding_window() >= 1
    assert shim.install_inference() >= 2


def reinit(module, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    with torch.no_grad():
        for p in module.parameters():
            if p.dim() > 1:
                p.copy_((torch.randn(p.shape, generator=g, device="cuda") * 0.02).to(p.dtype))


def err(a, b):
    e = (a.float() - b.float()).abs()
    return float(e.max()), float(e.mean()), float(b.float().pow(2).mean().sqrt())


@pytest.mark.parametrize("compress_type,topk", [("weightedpool", 48), ("weightedpool", 8), ("linear", 8)])
def test_nsa_layer_forward_backward_on_shim(ref, compress_type, topk):
    """topk 48 selects every block of these sequences: no element may leave the bound.  With topk 8 (configuration 4's value)
    and the N(0, 0.02) weights that configuration prescribes, the logits are tiny, attention is close to uniform and the
    block scores of a token differ by less than rounding: the two implementations legitimately choose different blocks for
    many tokens (the 1e-3 tie rule), which moves those tokens' rows.  That run is held to a mean bound only."""
    from native_sparse_attention.module import NativeSparseAttention
    import native_sparse_attention.module.native_sparse_attention as layer_mod
    import native_sparse_attention_triton_b200 as pkg

    if compress_type == "linear":
        # where the reference's Triton linear_compress does not compile (Triton 3.6 on sm_100), its layer runs on the
        # reference's own torch implementation of that operator; everything else of the reference side is untouched
        layer_mod.COMPRESS_TYPE_TO_FUNC["linear"] = refbox.reference_linear_compress()[0]
    cfg = dict(compress_type=compress_type, hidden_size=1024, num_q_heads=32, num_kv_heads=2, head_dim=128, kernel_size=32,
               kernel_stride=16, block_size=64, topk=topk, init_blocks=1, local_blocks=2, window_size=512,
               rope_config=refbox.llama3_rope_config(ref, 128, 4.0))
    torch.manual_seed(0)
    layer_ref = NativeSparseAttention(**cfg).cuda().to(torch.bfloat16)
    reinit(layer_ref, 5)
    seqlens = [700, 1900, 3000]
    cu = torch.tensor([0] + torch.tensor(seqlens).cumsum(0).tolist(), dtype=torch.int32, device="cuda")
    g = torch.Generator(device="cuda").manual_seed(9)
    x = torch.randn(sum(seqlens), 1024, generator=g, device="cuda").to(torch.bfloat16)
    dy = torch.randn(sum(seqlens), 1024, generator=g, device="cuda").to(torch.bfloat16)

    def run(layer):
        xi = x.clone().requires_grad_(True)
        y = layer(xi, cu)
        y.backward(dy)
        return y.detach(), xi.grad, {n: p.grad.clone() for n, p in layer.named_parameters() if p.grad is not None}

    y_r, dx_r, gr_r = run(layer_ref)
    before = pkg._lib.launch_count()
    use_this_package()
    layer = NativeSparseAttention(**cfg).cuda().to(torch.bfloat16)
    layer.load_state_dict(layer_ref.state_dict())
    assert layer.compress_func is {"linear": pkg.ops.linear_compress, "weightedpool": pkg.ops.weightedpool_compress}[compress_type]
    y, dx, gr = run(layer)
    assert pkg._lib.launch_count() - before >= 20, "the layer did not run on libnsa_b200.so"
    assert pkg.device_status() == 0
    rows = [("y", y, y_r), ("dx", dx, dx_r)] + [("d_" + n, gr[n], gr_r[n]) for n in sorted(gr_r)]
    for name, a, b in rows:
        # every tensor here is a sum over 1024-4096 products of 16-bit numbers: errors are judged on the tensor's own scale
        e = (a.float() - b.float()).abs()
        rms = max(float(b.float().pow(2).mean().sqrt()), 1e-6)
        rel = (e / b.float().abs().clamp(min=rms)).flatten()
        worst, mean = float(rel.max()), float(e.mean()) / rms
        q999 = float(rel.kthvalue(max(1, int(rel.numel() * 0.999))).values)
        print(f"layer {compress_type} topk {topk} {name}: max {worst:.4f} 99.9% {q999:.4f} mean {mean:.5f} (units of rms {rms:.4f})")
        if topk == 48:
            assert mean <= 1e-2 and q999 <= 0.1 and worst <= 0.25, (name, worst, q999, mean)
        else:
            assert mean <= 3e-2, (name, worst, q999, mean)


@pytest.mark.parametrize("topk", [16, 8])
def test_toy_nsa_llama_generate_on_shim(ref, topk):
    """topk 16 selects every block of these prompts, so the logits must agree at every step; with topk 8 (configuration
    5's value) a block whose score ties with another's within rounding can be chosen differently by the two
    implementations, which moves that step's logits: at most one step in six may leave the tight bound."""
    from native_sparse_attention.model import InferenceConfig, ToyNSALlama, ToyNSALlamaConfig
    import native_sparse_attention_triton_b200 as pkg

    cfg = ToyNSALlamaConfig(vocab_size=2048, hidden_size=1024, intermediate_size=2048, num_hidden_layers=2,
                            num_attention_heads=16, num_key_value_heads=1, head_dim=128, compress_type="weightedpool",
                            kernel_size=32, kernel_stride=16, block_size=64, topk=topk, init_blocks=1, local_blocks=2, window_size=512)
    icfg = InferenceConfig(max_batch_size=2, max_length=1024, max_new_tokens=12)
    torch.manual_seed(0)
    model_ref = ToyNSALlama(cfg, icfg).cuda().bfloat16()
    reinit(model_ref, 6)
    seqlens = [333, 800]
    cu = torch.tensor([0] + torch.tensor(seqlens).cumsum(0).tolist(), dtype=torch.int32, device="cuda")
    g = torch.Generator(device="cuda").manual_seed(10)
    ids = torch.randint(0, cfg.vocab_size, (sum(seqlens),), generator=g, device="cuda")
    steps = 12
    # the reference generates; its tokens are then fed to both models step by step so that the logits stay comparable
    logits_ref, tokens = [], []
    inp = ids
    for step in range(steps):
        lg = model_ref.inference(inp, cu, step)
        logits_ref.append(lg)
        inp = lg.argmax(-1)
        tokens.append(inp)
    before = pkg._lib.launch_count()
    use_this_package()
    model = ToyNSALlama(cfg, icfg).cuda().bfloat16()
    model.load_state_dict(model_ref.state_dict())
    agree, loose = 0, 0
    inp = ids
    for step in range(steps):
        lg = model.inference(inp, cu, step)
        mx, mean, rms = err(lg, logits_ref[step])
        print(f"model topk {topk} step {step}: logits max {mx:.5f} mean {mean:.6f} rms(ref) {rms:.5f}")
        assert mx <= 0.5 * rms and mean <= 5e-2 * rms, (step, mx, mean, rms)
        loose += not (mx <= 0.1 * rms and mean <= 1.5e-2 * rms)
        agree += int((lg.argmax(-1) == tokens[step]).sum())
        inp = tokens[step]
    assert loose <= (0 if topk == 16 else steps // 6), loose
    from native_sparse_attention_triton_b200.kv_cache import NSACache
    assert isinstance(model.kv_cache[0], NSACache)
    assert pkg._lib.launch_count() - before >= 100, "generation did not run on libnsa_b200.so"
    assert pkg.device_status() == 0
    print(f"greedy tokens equal to the reference's: {agree}/{steps * len(seqlens)}")
    # full generate() through the public call, for shape and for running at all
    out = model.generate(ids, cu, 4)
    assert out.shape == (len(seqlens), 4)
