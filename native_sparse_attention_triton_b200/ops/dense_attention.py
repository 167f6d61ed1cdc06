"""Dense varlen GQA attention with a strided-causal mask: shared by compressed_attention and
flash_attention_varlen.  Forward returns (o, lse) with lse fp32 [total_q, num_q_heads] in base 2."""
import torch

from .. import _lib
from ._common import dtype_code, ptr, stream_ptr


def varlen_attention_forward(q, k, v, cu_q, cu_k, max_seqlen_q, causal, window, stride, sm_scale):
    total_q, num_q_heads, head_dim = q.shape
    total_k, num_kv_heads, _ = k.shape
    batch = cu_q.shape[0] - 1
    if total_k == 0:
        return torch.zeros_like(q), torch.full((total_q, num_q_heads), float("-inf"), dtype=torch.float32, device=q.device)
    o = torch.empty(total_q, num_q_heads, head_dim, dtype=q.dtype, device=q.device)
    lse = torch.empty(total_q, num_q_heads, dtype=torch.float32, device=q.device)
    strides = _lib.strides_array(q.stride(0), q.stride(1), k.stride(0), k.stride(1), v.stride(0), v.stride(1),
                                 o.stride(0), o.stride(1))
    torch.cuda.set_device(q.device)
    rc = _lib.lib().nsa_varlen_attn_fwd(ptr(q), ptr(k), ptr(v), ptr(cu_q), ptr(cu_k), ptr(o), ptr(lse), total_q, total_k,
                                        batch, int(max_seqlen_q), num_q_heads, num_kv_heads, head_dim, int(bool(causal)),
                                        int(window), int(stride), strides, float(sm_scale), dtype_code(q),
                                        stream_ptr(q.device))
    _lib.check(rc, "nsa_varlen_attn_fwd")
    return o, lse


def varlen_attention_backward(q, k, v, o, lse, do, cu_q, cu_k, max_seqlen_q, max_seqlen_k, causal, window, stride,
                              sm_scale):
    from .attention_bwd import dense_attention_backward
    return dense_attention_backward(q, k, v, o, lse, do, cu_q, cu_k, max_seqlen_q, max_seqlen_k, causal, window,
                                    stride, sm_scale)
