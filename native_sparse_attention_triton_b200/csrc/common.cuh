// Device-side primitives shared by every kernel of the library (sm_100a only).
//
//  * dtype traits for the two supported storage types (bf16, fp16)
//  * warp-level tensor-core primitives (ldmatrix, mma.sync m16n8k16, movmatrix)
//  * mbarrier + TMA (cp.async.bulk.tensor) wrappers with BOUNDED waits: a wait that
//    does not complete within a clock budget records an error code in a global
//    status word and returns, so a broken pipeline can never hang the GPU.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nsa {

// ----------------------------------------------------------------------------------------
// status word: 0 = ok; kernels OR error bits into it, the host entry point reads it lazily.
// ----------------------------------------------------------------------------------------
enum : int {
  kErrWaitTimeout = 1,   // a bounded mbarrier wait gave up
  kErrBadIndex = 2,      // an index read from memory was outside its legal range
  kErrSmemLayout = 4,    // the dynamic shared-memory base is not aligned as the kernel's tile layout needs
};

struct Status {
  int* word;  // device pointer (may be nullptr)
  __device__ __forceinline__ void raise(int code) const {
    if (word) atomicOr(word, code);
  }
};

// ----------------------------------------------------------------------------------------
// dtype traits
// ----------------------------------------------------------------------------------------
template <typename T>
struct DT;

template <>
struct DT<__nv_bfloat16> {
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) {
    __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
    return __bfloat1622float2(v);
  }
  static __device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ __nv_bfloat16 from_float(float x) { return __float2bfloat16_rn(x); }
  static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  static constexpr CUtensorMapDataType kTmapType = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
};

template <>
struct DT<__half> {
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) {
    __half2 v = *reinterpret_cast<__half2*>(&u);
    return __half22float2(v);
  }
  static __device__ __forceinline__ float to_float(__half x) { return __half2float(x); }
  static __device__ __forceinline__ __half from_float(float x) { return __float2half_rn(x); }
  static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  static constexpr CUtensorMapDataType kTmapType = CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
};

// ----------------------------------------------------------------------------------------
// small helpers
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));  // pure: the compiler may schedule many of them back to back
  return y;
}

// 2^x where `keep` holds, else 0.  The exponential is evaluated unconditionally and the result selected, so a
// per-thread mask never turns into a divergent branch around the MUFU instruction.
__device__ __forceinline__ float masked_exp2(bool keep, float x) {
  const float e = fast_exp2(x);
  return keep ? e : 0.f;
}

// Packed fp32 pairs (sm_100: one instruction for two lanes of FMA / MUL).  The softmax threads of the tcgen05 kernels are
// bound by issue slots they share with the MMA-issuing warp, so halving their elementwise instruction count matters.
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("{\n .reg .b64 ra, rb, rc, rd;\n mov.b64 ra, {%2, %3};\n mov.b64 rb, {%4, %5};\n mov.b64 rc, {%6, %7};\n"
      " fma.rn.f32x2 rd, ra, rb, rc;\n mov.b64 {%0, %1}, rd;\n}\n"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return d;
}
__device__ __forceinline__ float2 fmul2(float2 a, float2 b) {
  float2 d;
  asm("{\n .reg .b64 ra, rb, rd;\n mov.b64 ra, {%2, %3};\n mov.b64 rb, {%4, %5};\n mul.rn.f32x2 rd, ra, rb;\n mov.b64 {%0, %1}, rd;\n}\n"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}

__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
  float2 d;
  asm("{\n .reg .b64 ra, rb, rd;\n mov.b64 ra, {%2, %3};\n mov.b64 rb, {%4, %5};\n add.rn.f32x2 rd, ra, rb;\n mov.b64 {%0, %1}, rd;\n}\n"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
// 2^x for a pair of fp32 values on the FMA pipe instead of the special-function unit (which delivers 16 results per clock
// per SM and bounds the softmax of a 128 x 128 tile at 1024 clocks): round to the nearest integer n with the 1.5 * 2^23
// trick, evaluate a cubic on f = x - n in [-0.5, 0.5] (relative error 7.5e-5, far below the 2^-9 or 2^-11 rounding the
// result gets when it is stored as a 16-bit probability), add n to the exponent field.  Inputs below -126 give about 1e-38.
__device__ __forceinline__ float2 exp2_poly2(float2 x) {
  const float2 magic = make_float2(12582912.f, 12582912.f);
  x.x = fmaxf(x.x, -126.f);
  x.y = fmaxf(x.y, -126.f);
  const float2 t = fadd2(x, magic);
  const float2 r = fadd2(t, make_float2(-12582912.f, -12582912.f));
  const float2 f = ffma2(r, make_float2(-1.f, -1.f), x);
  float2 q = ffma2(f, make_float2(0.0551716648f, 0.0551716648f), make_float2(0.2426111251f, 0.2426111251f));
  q = ffma2(q, f, make_float2(0.6932609677f, 0.6932609677f));
  q = ffma2(q, f, make_float2(0.9999280572f, 0.9999280572f));
  return make_float2(__int_as_float(__float_as_int(q.x) + (__float_as_int(t.x) << 23)),
                     __int_as_float(__float_as_int(q.y) + (__float_as_int(t.y) << 23)));
}
// Three-input maximum (one instruction on sm_100).
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;\n" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

__device__ __forceinline__ int lane_id() { return threadIdx.x & 31; }

// largest b such that cu[b] <= n (cu has nseq+1 ascending entries, cu[0] = 0)
__device__ __forceinline__ int find_sequence(const int* __restrict__ cu, int nseq, int n) {
  int lo = 0, hi = nseq;  // invariant: cu[lo] <= n < cu[hi]
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (__ldg(cu + mid) <= n) lo = mid; else hi = mid;
  }
  return lo;
}

// ----------------------------------------------------------------------------------------
// ldmatrix / movmatrix
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}

// ----------------------------------------------------------------------------------------
// 128-byte swizzled shared-memory tiles as written by TMA (CU_TENSOR_MAP_SWIZZLE_128B).
// A tile is a stack of "panels"; one panel holds ROWS rows of 64 16-bit elements (128 B
// per row) and must start on a 1024-byte boundary.  Element (row, col) of the logical
// [ROWS x (64*panels)] tile lives in panel col/64, at byte
//     row*128 + ((chunk ^ (row & 7)) << 4) + (col & 7)*2,   chunk = (col & 63) >> 3.
// ----------------------------------------------------------------------------------------
template <int ROWS>
__device__ __forceinline__ uint32_t swz_addr(uint32_t tile_base, int row, int chunk16 /* 16-byte chunk index over the full row */) {
  int panel = chunk16 >> 3;
  int c = chunk16 & 7;
  return tile_base + panel * (ROWS * 128) + row * 128 + ((c ^ (row & 7)) << 4);
}

// ----------------------------------------------------------------------------------------
// mbarrier + TMA
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}

// Non-blocking test of a phase: unlike try_wait, which may suspend the thread for a system-dependent time when the phase
// is not complete, this returns at once.  For threads that poll several barriers and must not sleep on one of them.
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}

// Bounded wait: gives up after ~2^30 SM clocks (about half a second), raising kErrWaitTimeout.
// Once any thread of the grid has given up, every later wait returns at once, so a broken
// pipeline costs one timeout in total, not one per wait.  Returns false on timeout; the caller
// keeps going (results are garbage, the status word says so).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const Status& st) {
  if (mbar_try_wait(bar, parity)) return true;
  long long t0 = clock64();
  int spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if (((++spins) & 255) == 0) {
      if (st.word && (*reinterpret_cast<volatile int*>(st.word) & kErrWaitTimeout)) return false;
      if ((clock64() - t0) > (1ll << 30)) {
        st.raise(kErrWaitTimeout);
        return false;
      }
    }
  }
  return true;
}

// 3-D tiled TMA load, coordinates innermost first.  c0 * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* tm, uint64_t* bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];\n"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(tm)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* tm, uint64_t* bar, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];\n"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(tm)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// 3-D tiled TMA store of a shared-memory tile (written through the generic proxy: fence_proxy_async() and a barrier first).
// Coordinates as for the load; never negative.  Completion is tracked per thread in bulk groups.
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* tm, const void* src, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];\n"
               ::"l"(reinterpret_cast<uint64_t>(tm)), "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;\n" ::: "memory"); }
// the committed stores have read their shared-memory source (it may be reused or released)
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory"); }
// start moving a 3-D tile into L2 only (no shared-memory destination, no completion tracking)
__device__ __forceinline__ void tma_prefetch_l2_3d(const CUtensorMap* tm, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];\n" ::"l"(reinterpret_cast<uint64_t>(tm)),
               "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tm) {
  asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(tm)) : "memory");
}

// ----------------------------------------------------------------------------------------
// cp.async (16-byte, L2-only) for tiles whose rows are gathered with computed addresses
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool pred) {
  const int sz = pred ? 16 : 0;  // 0 -> the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// ----------------------------------------------------------------------------------------
// warp reductions over the 4 lanes that share one fragment row
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ float quad_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
  return v;
}
__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  return v;
}

}  // namespace nsa
