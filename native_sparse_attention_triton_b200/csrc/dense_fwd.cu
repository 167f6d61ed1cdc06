// Forward of dense varlen GQA attention with a strided-causal mask:
//     query at in-sequence position t sees key i  iff  t >= i*stride + (window - 1).
// window = 32, stride = 16 gives attention over compressed keys (compressed_attention);
// window = stride = 1 gives ordinary causal attention; causal = 0 gives full attention.
//
// Argument checks and the C entry points; the kernel (tcgen05) is in dense_fwd_tc.cu.

#include "attn_tile.cuh"
#include "dispatch.h"
#include "host_util.h"
#include "nsa_b200.h"

namespace nsa {

struct DenseFwdParams {
  const void* q;
  void* o;
  float* lse;  // [Nq, Hq]
  const int* cu_q;
  const int* cu_k;
  long long q_sn, q_sh, o_sn, o_sh;
  int B, Hq, Hkv, G, logG;
  int window, stride, causal;
  float scale2;
  Status st;
};

// tcgen05 implementation (dense_fwd_tc.cu)
int varlen_attn_fwd_tc(const void* q, const void* k, const void* v, const int* cu_q, const int* cu_k, void* o, float* lse,
                       int total_q, int total_k, int batch, int max_seqlen_q, int Hq, int Hkv, int head_dim, int causal,
                       int window, int stride, int left, const long long* strides, float sm_scale, int dtype, cudaStream_t stream);

}  // namespace nsa

// left >= 0 adds the lower bound key >= t - left (sliding window); only with the plain causal mask and on the tcgen05 kernel
static int varlen_attn_fwd_common(const void* q, const void* k, const void* v, const int* cu_seqlens_q,
                                  const int* cu_seqlens_k, void* o, float* lse, int total_q, int total_k, int batch,
                                  int max_seqlen_q, int num_q_heads, int num_kv_heads, int head_dim, int causal,
                                  int window, int stride, int left, const long long* strides, float sm_scale, int dtype,
                                  void* stream) {
  using namespace nsa;
  if (left >= 0 && (!causal || window != 1 || stride != 1)) return kUnsupported;
  if (!q || !cu_seqlens_q || !cu_seqlens_k || !o || !lse || !strides) return kInvalid;
  if (total_q <= 0 || batch <= 0 || max_seqlen_q <= 0 || num_kv_heads <= 0 || num_q_heads % num_kv_heads) return kInvalid;
  if (window < 1 || stride < 1) return kInvalid;
  const int G = num_q_heads / num_kv_heads;
  if (G > 16 || (G & (G - 1))) return kUnsupported;
  if (total_k <= 0) {  // no key anywhere: outputs are zero, lse = -inf (caller pre-fills); nothing to launch
    return kOk;
  }
  if (!k || !v) return kInvalid;
  DenseFwdParams p;
  p.q = q; p.o = o; p.lse = lse; p.cu_q = cu_seqlens_q; p.cu_k = cu_seqlens_k;
  p.q_sn = strides[0]; p.q_sh = strides[1]; p.o_sn = strides[6]; p.o_sh = strides[7];
  p.B = batch; p.Hq = num_q_heads; p.Hkv = num_kv_heads; p.G = G;
  p.logG = 0;
  while ((1 << p.logG) < G) ++p.logG;
  p.window = window; p.stride = stride; p.causal = causal;
  p.scale2 = sm_scale * kLog2e;
  p.st.word = status_word();
  if ((p.q_sn | p.q_sh | p.o_sn | p.o_sh) % 8 || !aligned16(q) || !aligned16(o)) return kInvalid;
  return varlen_attn_fwd_tc(q, k, v, cu_seqlens_q, cu_seqlens_k, o, lse, total_q, total_k, batch, max_seqlen_q, num_q_heads,
                            num_kv_heads, head_dim, causal, window, stride, left, strides, sm_scale, dtype,
                            static_cast<cudaStream_t>(stream));
}

extern "C" int nsa_varlen_attn_fwd(const void* q, const void* k, const void* v, const int* cu_seqlens_q,
                                   const int* cu_seqlens_k, void* o, float* lse, int total_q, int total_k, int batch,
                                   int max_seqlen_q, int num_q_heads, int num_kv_heads, int head_dim, int causal,
                                   int window, int stride, const long long* strides, float sm_scale, int dtype,
                                   void* stream) {
  return varlen_attn_fwd_common(q, k, v, cu_seqlens_q, cu_seqlens_k, o, lse, total_q, total_k, batch, max_seqlen_q, num_q_heads,
                                num_kv_heads, head_dim, causal, window, stride, -1, strides, sm_scale, dtype, stream);
}

extern "C" int nsa_window_attn_fwd(const void* q, const void* k, const void* v, const int* cu_seqlens, void* o, float* lse,
                                   int total_len, int batch, int max_seqlen, int num_q_heads, int num_kv_heads, int head_dim,
                                   int window_left, const long long* strides, float sm_scale, int dtype, void* stream) {
  if (window_left < 0) return nsa::kInvalid;
  return varlen_attn_fwd_common(q, k, v, cu_seqlens, cu_seqlens, o, lse, total_len, total_len, batch, max_seqlen, num_q_heads,
                                num_kv_heads, head_dim, 1, 1, 1, window_left, strides, sm_scale, dtype, stream);
}
