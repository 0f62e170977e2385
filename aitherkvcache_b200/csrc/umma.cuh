// tcgen05 (5th-generation tensor core) helpers shared by the encode and decode kernels:
// shared-memory matrix descriptors for K-major 16-bit operands in the 128-byte-swizzled
// layout, MMA issue / commit, tensor-memory loads and a bounded mbarrier wait.
//
// Operand layout (128 rows x 128 K-elements of 16 bits = 32 KB, base 1024-byte aligned):
// two halves of 64 K-elements; in a half, row r is 128 bytes at r*128 and its 16-byte
// chunk c is stored at chunk c ^ (r & 7).  One MMA consumes 16 K-elements (32 bytes of
// every row): K-step kk of a half starts 32*kk bytes into the rows.
#pragma once

#include "common.cuh"

namespace akv {

constexpr int TC_HALF_BYTES = 128 * 128;          // 128 rows x 64 16-bit elements (one swizzle atom wide)
constexpr int TC_OPER_BYTES = 2 * TC_HALF_BYTES;  // a 128 x 128 16-bit operand
constexpr int TC_SPIN_LIMIT = 1 << 17;            // tries of one mbarrier wait before giving up ...
constexpr long long TC_WAIT_CYCLES = 1ll << 27;   // ... or this many SM cycles (tens of milliseconds), whichever comes first

// Byte offset of element (row, k) inside an operand.
__device__ __forceinline__ uint32_t tc_operand_offset(int row, int k) {
  return (uint32_t)((k >> 6) * TC_HALF_BYTES + row * 128 + (((((k & 63) >> 3) ^ (row & 7)) << 4) | ((k & 7) << 1)));
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

// K-major operand, 128-byte swizzle: rows 128 B apart, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      :: "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

__device__ __forceinline__ void umma_commit(uint32_t mbar_s) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               :: "r"(mbar_s) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr) : "memory");
}

__device__ __forceinline__ bool mbar_wait(uint32_t mbar_s, uint32_t parity) {
  const long long t0 = clock64();
  for (int it = 0; it < TC_SPIN_LIMIT; ++it) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(done) : "r"(mbar_s), "r"(parity) : "memory");
    if (done) return true;
    if ((it & 15) == 15 && clock64() - t0 > TC_WAIT_CYCLES) break;
  }
  return false;
}

__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}

__device__ __forceinline__ uint32_t bswap32(uint32_t v) { return __byte_perm(v, 0u, 0x0123); }

}  // namespace akv
