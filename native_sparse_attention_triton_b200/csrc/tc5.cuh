// 5th-generation tensor core primitives (tcgen05): shared-memory matrix descriptors, instruction
// descriptors, MMA issue / commit, tensor-memory (TMEM) allocation and access.
//
// Operand tiles are the 128-byte-swizzled panels TMA writes (see swz_addr in common.cuh):
//   K-major operand  (rows = M or N index, 64 contiguous K elements = one 128 B row of a panel):
//       8-row groups are 1024 B apart (stride byte offset); a K step of 16 elements advances the start address by 32 B.
//   MN-major operand (rows = K index, 64 contiguous M/N elements per panel row):
//       8-row (K) groups are 1024 B apart (stride byte offset); the next 64 M/N elements live in the next panel
//       (leading byte offset = panel size); a K step of 16 rows advances the start address by 2048 B.
#pragma once
#include "common.cuh"

namespace nsa {

// ---- shared-memory matrix descriptor (SWIZZLE_128B) ----
__device__ __forceinline__ uint64_t umma_desc_kmajor(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ uint64_t umma_desc_mnmajor(uint32_t saddr, uint32_t panel_bytes) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)((panel_bytes >> 4) & 0x3FFF) << 16) |
         ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

// ---- instruction descriptor: fp32 accumulate, 16-bit inputs ----
template <typename T>
__device__ __forceinline__ constexpr uint32_t umma_idesc(int M, int N, bool a_mn_major, bool b_mn_major) {
  const uint32_t fmt = (sizeof(T) == 2 && DT<T>::kTmapType == CU_TENSOR_MAP_DATA_TYPE_BFLOAT16) ? 1u : 0u;
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) |
         ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread
__device__ __forceinline__ void umma_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, bool accumulate) {
  const uint32_t acc = accumulate ? 1u : 0u;
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(acc)
      : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]: A is read from tensor memory (lane = row, each 32-bit column = two consecutive
// 16-bit K elements), which spares the shared-memory bandwidth an SMEM A operand costs.  Issued by ONE thread.
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, bool accumulate) {
  const uint32_t acc = accumulate ? 1u : 0u;
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(acc)
      : "memory");
}

// ---- blocks of MMAs over the reduction dimension ----
// How to issue (measured on B200 with blocks of 8 MMAs of 128x128x16, a commit and a barrier test between blocks):
// the queue in front of the tensor pipe is shallow, so every instruction the issuing thread executes between two MMAs
// is time the pipe waits.  The whole warp must run the control flow CONVERGED, with only the MMA and commit
// instructions under elect_one(), and descriptors must be built from (warp-uniform) addresses at each use: the
// compiler then keeps all of that arithmetic in the uniform datapath and the block runs at 64 clocks per MMA, the pipe's
// rate.  The same code inside `if (lane == 0)` takes 91 clocks per MMA.
// D = A B^T, both operands K-major SMEM tiles made of [rows][64-element] panels PANEL bytes apart; NK steps of 16.
template <int NK, int PANEL>
__device__ __forceinline__ void umma_block_ss(uint32_t d_tmem, uint32_t a_addr, uint32_t b_addr, uint32_t idesc) {
#pragma unroll
  for (int kk = 0; kk < NK; ++kk) {
    const uint32_t off = (kk >> 2) * PANEL + (kk & 3) * 32;
    umma_ss(d_tmem, umma_desc_kmajor(a_addr + off), umma_desc_kmajor(b_addr + off), idesc, kk > 0);
  }
}
// D (+)= A B with A in TMEM as 16-bit pairs written by threads that own 64 source columns each (reduction step kk
// sits at column 64*(kk/4) + 8*(kk%4) of the A region) and B an MN-major SMEM tile (16 reduction rows = 2048 bytes,
// 64-element panels PANEL bytes apart).
template <int NK, int PANEL>
__device__ __forceinline__ void umma_block_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_addr, uint32_t idesc, bool accumulate) {
  umma_ts(d_tmem, a_tmem, umma_desc_mnmajor(b_addr, PANEL), idesc, accumulate);
#pragma unroll
  for (int kk = 1; kk < NK; ++kk)
    umma_ts(d_tmem, a_tmem + 64 * (kk >> 2) + 8 * (kk & 3), umma_desc_mnmajor(b_addr + kk * 2048, PANEL), idesc, true);
}

// the mbarrier gets one arrival when every MMA issued so far by this thread has completed
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }

// ---- TMEM allocation (one full warp executes these) ----
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(smem_dst)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(ncols) : "memory");
}

// ---- TMEM <-> registers: each thread of a warp reads/writes 32 consecutive 32-bit columns of its own lane ----
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
// 16 consecutive 32-bit columns of the thread's own lane
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};\n"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

// TMEM address of (lane, column) relative to an allocation base
__device__ __forceinline__ uint32_t tmem_addr(uint32_t base, int lane, int col) { return base + ((uint32_t)lane << 16) + (uint32_t)col; }

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}\n" : "=r"(pred));
  return pred != 0;
}

}  // namespace nsa
