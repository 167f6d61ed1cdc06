// Rotary position embedding of a varlen batch, forward and backward, in one pass over HBM.
//
//   y[n, h, :d/2] = x1 * cos - x2 * sin,   y[n, h, d/2:] = x2 * cos + x1 * sin,   (x1, x2) = the two halves of x[n, h, :]
//   angle[j] = inv_freq[j] * position(n),  cos/sin scaled by attention_scaling and rounded to the tensor's dtype
//
// This is x * cos + rotate_half(x) * sin of native_sparse_attention/module/rope.py:36-41,204-209 with the tables of
// generate_cos_sin (:126-155, fp32 angle = inv_freq * position, cos/sin rounded to x.dtype) and the positions of
// generate_pos_embs (:158-195): prefill (step 0) token t of its sequence sits at t * stride; decode (step > 0) row b sits
// at (seqlen_b + step - 1) * stride.  The reference builds the tables with a Python loop over the batch, three
// elementwise passes and a concatenation; here positions come from cu_seqlens on the device, each CTA computes the
// cos/sin of a few tokens once into shared memory and every thread rotates 8 + 8 elements per 16-byte load pair.
// The backward pass is the same rotation by the opposite angle.
#include "common.cuh"
#include "dispatch.h"
#include "host_util.h"
#include "nsa_b200.h"

namespace nsa {

struct RopeParams {
  const void* x;
  void* y;
  const float* inv_freq;  // [D / 2]
  const int* cu;          // [B + 1] cu_seqlens, or [B] lengths when step < 0
  long long x_sn, x_sh, y_sn, y_sh;
  int N, B, H, step, stride, inverse;
  float scaling;
};

__device__ __forceinline__ uint4 ld16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

template <typename T, int D>
__device__ __forceinline__ void rope_rows(const RopeParams& p, int first_block, int num_blocks) {
  constexpr int HALF = D / 2;
  constexpr int TOK = 256 / HALF;  // tokens whose tables one CTA holds at a time
  constexpr int CH = HALF / 8;     // 16-byte chunks per half row
  __shared__ float cs[TOK][HALF], sn[TOK][HALF];
  const int tid = threadIdx.x;
  for (int tok0 = first_block * TOK; tok0 < p.N; tok0 += num_blocks * TOK) {
    {
      const int tl = tid / HALF, j = tid % HALF, n = tok0 + tl;
      if (n < p.N) {
        int pos;
        if (p.step == 0) {
          const int b = find_sequence(p.cu, p.B, n);
          pos = (n - __ldg(p.cu + b)) * p.stride;
        } else if (p.step > 0) {
          pos = (__ldg(p.cu + n + 1) - __ldg(p.cu + n) + p.step - 1) * p.stride;
        } else {  // decode row at a length counter read from the device
          pos = __ldg(p.cu + n) * p.stride;
        }
        float s, c;
        sincosf(__ldg(p.inv_freq + j) * (float)pos, &s, &c);
        c = DT<T>::to_float(DT<T>::from_float(c * p.scaling));
        s = DT<T>::to_float(DT<T>::from_float(s * p.scaling));
        cs[tl][j] = c;
        sn[tl][j] = p.inverse ? -s : s;
      }
    }
    __syncthreads();
    const int per_tok = p.H * CH;
    for (int it = tid; it < TOK * per_tok; it += 256) {
      const int tl = it / per_tok, rem = it % per_tok, h = rem / CH, c = rem % CH;
      const int n = tok0 + tl;
      if (n >= p.N) break;
      const T* xp = static_cast<const T*>(p.x) + (long long)n * p.x_sn + (long long)h * p.x_sh + c * 8;
      const uint4 a = ld16(xp), b = ld16(xp + HALF);
      uint4 ya, yb;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float2 x1 = DT<T>::unpack(reinterpret_cast<const uint32_t*>(&a)[w]);
        const float2 x2 = DT<T>::unpack(reinterpret_cast<const uint32_t*>(&b)[w]);
        const float c0 = cs[tl][c * 8 + 2 * w], c1 = cs[tl][c * 8 + 2 * w + 1];
        const float s0 = sn[tl][c * 8 + 2 * w], s1 = sn[tl][c * 8 + 2 * w + 1];
        reinterpret_cast<uint32_t*>(&ya)[w] = DT<T>::pack(fmaf(x1.x, c0, -x2.x * s0), fmaf(x1.y, c1, -x2.y * s1));
        reinterpret_cast<uint32_t*>(&yb)[w] = DT<T>::pack(fmaf(x2.x, c0, x1.x * s0), fmaf(x2.y, c1, x1.y * s1));
      }
      T* yp = static_cast<T*>(p.y) + (long long)n * p.y_sn + (long long)h * p.y_sh + c * 8;
      *reinterpret_cast<uint4*>(yp) = ya;
      *reinterpret_cast<uint4*>(yp + HALF) = yb;
    }
    __syncthreads();
  }
}

template <typename T, int D>
__global__ void __launch_bounds__(256) rope_kernel(RopeParams p) {
  rope_rows<T, D>(p, blockIdx.x, gridDim.x);
}

// The three rotations of a decode step (query, key, compressed key) in one launch: blockIdx.y picks the tensor.
struct Rope3Params {
  RopeParams seg[3];
};
template <typename T, int D>
__global__ void __launch_bounds__(256) rope3_kernel(Rope3Params p) {
  rope_rows<T, D>(p.seg[blockIdx.y], blockIdx.x, gridDim.x);
}

template <typename T, int D>
static int launch_rope3(Rope3Params p, cudaStream_t stream) {
  constexpr int TOK = 256 / (D / 2);
  LaunchScope ls_("rope3", stream);
  rope3_kernel<T, D><<<dim3((p.seg[0].N + TOK - 1) / TOK, 3), 256, 0, stream>>>(p);
  return cuda_rc(cudaGetLastError());
}

template <typename T, int D>
static int launch_rope(RopeParams p, cudaStream_t stream) {
  constexpr int TOK = 256 / (D / 2);
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long want = ((long long)p.N + TOK - 1) / TOK;
  const long long cap = (long long)sms * 8;  // 8 resident CTAs of 256 threads per SM
  LaunchScope ls_("rope", stream);
  rope_kernel<T, D><<<(int)(want < cap ? want : cap), 256, 0, stream>>>(p);
  return cuda_rc(cudaGetLastError());
}

}  // namespace nsa

extern "C" int nsa_rope(const void* x, void* y, const float* inv_freq, const int* cu_seqlens, int total_rows, int batch,
                        int num_heads, int head_dim, int step, int stride, float attention_scaling, int inverse,
                        long long x_stride_n, long long x_stride_h, long long y_stride_n, long long y_stride_h, int dtype,
                        void* stream) {
  using namespace nsa;
  if (!inv_freq || !cu_seqlens || total_rows < 0 || batch <= 0 || num_heads <= 0 || step < 0 || stride <= 0) return kInvalid;
  if (step > 0 && total_rows != batch) return kInvalid;  // decode: one row per sequence
  if (total_rows == 0) return kOk;
  if (!x || !y || !aligned16(x) || !aligned16(y)) return kInvalid;
  if ((x_stride_n | x_stride_h | y_stride_n | y_stride_h) % 8) return kInvalid;
  RopeParams p;
  p.x = x; p.y = y; p.inv_freq = inv_freq; p.cu = cu_seqlens;
  p.x_sn = x_stride_n; p.x_sh = x_stride_h; p.y_sn = y_stride_n; p.y_sh = y_stride_h;
  p.N = total_rows; p.B = batch; p.H = num_heads; p.step = step; p.stride = stride; p.inverse = inverse ? 1 : 0;
  p.scaling = attention_scaling;
  return NSA_DISPATCH_T_D(dtype, head_dim, launch_rope, p, static_cast<cudaStream_t>(stream));
}

extern "C" int nsa_rope_decode(const void* x, void* y, const float* inv_freq, const int* lengths, int batch, int num_heads,
                               int head_dim, int stride, float attention_scaling, int inverse, long long x_stride_n,
                               long long x_stride_h, long long y_stride_n, long long y_stride_h, int dtype, void* stream) {
  using namespace nsa;
  if (!inv_freq || !lengths || batch <= 0 || num_heads <= 0 || stride <= 0) return kInvalid;
  if (!x || !y || !aligned16(x) || !aligned16(y)) return kInvalid;
  if ((x_stride_n | x_stride_h | y_stride_n | y_stride_h) % 8) return kInvalid;
  RopeParams p;
  p.x = x; p.y = y; p.inv_freq = inv_freq; p.cu = lengths;
  p.x_sn = x_stride_n; p.x_sh = x_stride_h; p.y_sn = y_stride_n; p.y_sh = y_stride_h;
  p.N = batch; p.B = batch; p.H = num_heads; p.step = -1; p.stride = stride; p.inverse = inverse ? 1 : 0;
  p.scaling = attention_scaling;
  return NSA_DISPATCH_T_D(dtype, head_dim, launch_rope, p, static_cast<cudaStream_t>(stream));
}

extern "C" int nsa_rope_decode3(const void* q, void* yq, const void* k, void* yk, const void* ck, void* yck,
                                const float* inv_freq, const int* lengths_qk, const int* lengths_ck, int batch,
                                int num_q_heads, int num_kv_heads, int head_dim, int stride_ck, float attention_scaling,
                                const long long* strides, int dtype, void* stream) {
  using namespace nsa;
  if (!inv_freq || !lengths_qk || !lengths_ck || !strides || batch <= 0 || num_q_heads <= 0 || num_kv_heads <= 0 || stride_ck <= 0)
    return kInvalid;
  const void* x[3] = {q, k, ck};
  void* y[3] = {yq, yk, yck};
  Rope3Params p;
  for (int i = 0; i < 3; ++i) {
    if (!x[i] || !y[i] || !aligned16(x[i]) || !aligned16(y[i])) return kInvalid;
    const long long* st = strides + 4 * i;
    if ((st[0] | st[1] | st[2] | st[3]) % 8) return kInvalid;
    RopeParams& r = p.seg[i];
    r.x = x[i]; r.y = y[i]; r.inv_freq = inv_freq; r.cu = i == 2 ? lengths_ck : lengths_qk;
    r.x_sn = st[0]; r.x_sh = st[1]; r.y_sn = st[2]; r.y_sh = st[3];
    r.N = batch; r.B = batch; r.H = i == 0 ? num_q_heads : num_kv_heads; r.step = -1; r.stride = i == 2 ? stride_ck : 1;
    r.inverse = 0; r.scaling = attention_scaling;
  }
  return NSA_DISPATCH_T_D(dtype, head_dim, launch_rope3, p, static_cast<cudaStream_t>(stream));
}
