// Building blocks of the sm_100a kernels that use the 5th-generation tensor
// cores: mbarriers with bounded waits, TMA tensor loads, shared-memory matrix
// descriptors, tcgen05.mma / commit / ld, and the host-side lookup of the
// driver's tensor-map encoder.  Inline PTX; no library.
#pragma once
#include "common.cuh"
#include <cuda.h>

#define TG_SPIN_LIMIT (1u << 22)

__device__ __forceinline__ unsigned tg_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(void* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(tg_smem(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(void* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(tg_smem(bar)), "r"(bytes) : "memory");
}
// true when the phase with this parity has completed; false after the spin limit.  One look without
// blocking first: most waits of a pipeline in step find the phase complete, and test_wait then costs 100 to
// 200 cycles less than try_wait (stamped in the prompt attention: a passing wait 225 -> 133 cycles).
__device__ __forceinline__ bool mbar_wait(void* bar, unsigned parity, int* err) {
  const unsigned addr = tg_smem(bar);
  {
    unsigned done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    if (done) return true;
  }
  for (unsigned spin = 0; spin < TG_SPIN_LIMIT; ++spin) {
    unsigned done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    if (done) return true;
  }
  atomicOr(err, 16);
  return false;
}
// one look, no waiting
__device__ __forceinline__ bool mbar_test(void* bar, unsigned parity) {
  unsigned done;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
               "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(done) : "r"(tg_smem(bar)), "r"(parity) : "memory");
  return done != 0;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, void* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(tg_smem(dst)), "l"((unsigned long long)map), "r"(x), "r"(y), "r"(tg_smem(bar)) : "memory");
}
// K-major operand tile of rows x 64 bf16 with 128-byte swizzle: rows are 128 bytes, groups
// of 8 rows are 1024 bytes apart.  Fields: start address >> 4; leading byte offset 1
// (unused with swizzle); stride byte offset 1024 >> 4; version 1; layout type 2 (128B swizzle).
__device__ __forceinline__ unsigned long long umma_desc(const void* tile) {
  unsigned long long d = 0;
  d |= (unsigned long long)((tg_smem(tile) >> 4) & 0x3FFF);
  d |= (unsigned long long)1 << 16;
  d |= (unsigned long long)(1024 >> 4) << 32;
  d |= (unsigned long long)1 << 46;
  d |= (unsigned long long)2 << 61;
  return d;
}
__device__ __forceinline__ void umma_bf16(unsigned tmem_d, unsigned long long da, unsigned long long db,
                                          unsigned idesc, unsigned accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
               ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
               : "memory");
}
// The same with the A operand in tensor memory: row i of A in lane i, two bfloat16 of K a 32-bit column
// (what tcgen05.st.32x32b of packed pairs leaves there), from column ta on.
__device__ __forceinline__ void umma_bf16_tmem_a(unsigned tmem_d, unsigned ta, unsigned long long db,
                                                 unsigned idesc, unsigned accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %6, %7, %8}, p;\n\t}"
               ::"r"(tmem_d), "r"(ta), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
               : "memory");
}
__device__ __forceinline__ void umma_commit(void* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(tg_smem(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(unsigned taddr, unsigned* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
               "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                 "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                 "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
               : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st32(unsigned taddr, const unsigned* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
               "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                 "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                 "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                 "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
               : "memory");
}
__device__ __forceinline__ void tmem_st16(unsigned taddr, const unsigned* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
               "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                 "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(void* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tg_smem(bar)) : "memory");
}

// A K-major operand tile advanced by `bytes` along K inside its 128-byte swizzle atom, or by whole
// 1024-byte row groups: the address field counts 16 bytes.
__device__ __forceinline__ unsigned long long umma_desc_advance(unsigned long long desc, int bytes) {
  return desc + (unsigned long long)(bytes >> 4);
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
typedef CUresult (*tg_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static tg_encode_fn tg_get_encode() {
  static tg_encode_fn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (tg_encode_fn)p;
  }
  return fn;
}

