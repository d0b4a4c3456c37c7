// Blackwell (sm_100a) building blocks used by the tcgen05 kernels: mbarriers with bounded
// waits, TMA tile loads, TMEM allocation / load / store, UMMA shared-memory and instruction
// descriptors, and single-thread tcgen05.mma issue.
//
// Every wait in here is bounded by a cycle budget.  When a wait gives up it records a code in
// a CTA-wide abort flag and in the device-global status word; all later waits of the CTA return
// at once, the CTA drains, frees its TMEM and exits, and CTAs that start afterwards exit
// immediately.  The host reads the word through jvpfa_device_status().
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace jvpfa {
namespace tc5 {

constexpr long long kWaitBudgetCycles = 1ll << 31;  // about one second at B200 clocks

enum AbortCode : int {
  kAbortNone = 0,
  kAbortQFull = 1,
  kAbortKvFull = 2,
  kAbortKvEmpty = 3,
  kAbortSFull = 4,
  kAbortPFull = 5,
  kAbortOFull = 6,
  kAbortAux = 7,
  kAbortBwdOwn = 8,
  kAbortBwdLoopFull = 9,
  kAbortBwdLoopEmpty = 10,
  kAbortBwdSFull = 11,
  kAbortBwdPFull = 12,
  kAbortBwdDone = 13,
};

template <typename T>
struct Fmt;
template <>
struct Fmt<__nv_bfloat16> {
  static constexpr int kIdesc = 1;
  static constexpr CUtensorMapDataType kTma = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
};
template <>
struct Fmt<__half> {
  static constexpr int kIdesc = 0;
  static constexpr CUtensorMapDataType kTma = CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Two accumulator words as a packed pair of fp32 values, and the three-input maximum.
__device__ __forceinline__ float2 pf2(uint32_t a, uint32_t b) { return make_float2(__uint_as_float(a), __uint_as_float(b)); }
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

// Read-only global loads and 16-bit unpacking used for user masks and bias.
template <typename T>
__device__ __forceinline__ float2 unpack2(uint32_t w);
template <>
__device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t w) {
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
template <>
__device__ __forceinline__ float2 unpack2<__half>(uint32_t w) {
  return __half22float2(*reinterpret_cast<const __half2*>(&w));
}

// One 16-bit element (in the low half of h) as float.
template <typename T>
__device__ __forceinline__ float unpack1(uint32_t h);
template <>
__device__ __forceinline__ float unpack1<__nv_bfloat16>(uint32_t h) {
  return __uint_as_float(h << 16);
}
template <>
__device__ __forceinline__ float unpack1<__half>(uint32_t h) {
  return __half2float(__ushort_as_half((unsigned short)h));
}

__device__ __forceinline__ uint4 ldg_nc_v4(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
  return r;
}

__device__ __forceinline__ uint32_t ldg_nc_u8(const void* p) {
  uint32_t r;
  asm volatile("ld.global.nc.u8 %0, [%1];" : "=r"(r) : "l"(p));
  return r;
}
__device__ __forceinline__ uint32_t ldg_nc_u16(const void* p) {
  uint16_t r;
  asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(r) : "l"(p));
  return r;
}

// Host: (64, L, H, B) view of a 16-bit tensor whose batch / head / row strides (in elements) are given
// (all zero: (B,H,L,64) row-major); box = 64 columns x box_rows rows, 128-byte swizzle, out-of-range
// rows read as zero.  Defined in fwd_tc5.cu.
bool encode_map4(CUtensorMap* m, CUtensorMapDataType dt, const void* ptr, int L, int H, int B, const int64_t* stride_bhl,
                 int box_rows);
// The same for head dimension D (64-column boxes: a D = 128 tile is two loads).
bool encode_map4d(CUtensorMap* m, CUtensorMapDataType dt, const void* ptr, int D, int L, int H, int B, const int64_t* stride_bhl,
                  int box_rows);
// Row-major fp32 (B, H, L, D) tensor, 32-column boxes with 128-byte swizzle (target of TMA reductions).
bool encode_map4d_f32(CUtensorMap* m, const void* ptr, int D, int L, int H, int B, int box_rows);

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---- mbarrier ------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

struct AbortState {
  volatile int* cta_flag;  // shared memory
  int* global_status;      // device global
};

// Bounded wait.  Returns false (and latches the abort state) when the budget runs out or when
// another thread of the CTA has already given up.  A measured mbarrier hand-off between two warps
// costs ~200 cycles; reading the clock costs several tens of cycles, so the wait first polls
// without looking at it.  The budget and the abort flag are checked in the out-of-line part.
// First failure wins; the code also goes to the host-visible mirror whose device address sits beside the status word
// (two ints further, 8-byte aligned), so that the host learns of it without synchronising.
__device__ __forceinline__ void publish_abort(int* global_status, int code) {
  if (atomicCAS(global_status, 0, code) == 0) {
    int* mirror = *reinterpret_cast<int* const*>(global_status + 2);
    if (mirror) {
      *reinterpret_cast<volatile int*>(mirror) = code;
      __threadfence_system();
    }
  }
}
static __device__ __noinline__ bool mbar_wait_slow_u32(uint32_t bar, uint32_t parity, volatile int* cta_flag,
                                                       int* global_status, int code);
__device__ __forceinline__ bool mbar_try_wait_u32(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_u32(uint32_t bar, uint32_t parity, const AbortState& ab, int code) {
#pragma unroll 1
  for (int i = 0; i < 128; ++i)
    if (mbar_try_wait_u32(bar, parity)) return true;
  return mbar_wait_slow_u32(bar, parity, ab.cta_flag, ab.global_status, code);
}
// The general form.  Measured on the forward kernels (two CTAs per SM, many warps waiting at once):
// a poll loop that reads the clock right after the first failed attempt is ~5 % faster overall
// than the tight loop above, which takes issue slots from the warps that compute.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const AbortState& ab, int code) {
  const uint32_t addr = smem_u32(bar);
  if (mbar_try_wait_u32(addr, parity)) return true;
  const long long t0 = clock64();
  int polls = 0;
  while (true) {
    if (mbar_try_wait_u32(addr, parity)) return true;
    if ((++polls & 63) == 0) {
      if (*ab.cta_flag != 0) return false;
      if (clock64() - t0 > kWaitBudgetCycles) {
        *ab.cta_flag = code;
        publish_abort(ab.global_status, code);
        return false;
      }
    }
  }
}
// For roles far from the critical path (a producer several stages ahead): sleeps between attempts, because every
// attempt is an access on the shared-memory port that the MMA operands come through.
template <int NS = 128>
__device__ __forceinline__ bool mbar_wait_backoff(uint64_t* bar, uint32_t parity, const AbortState& ab, int code) {
  const uint32_t addr = smem_u32(bar);
  if (mbar_try_wait_u32(addr, parity)) return true;
  const long long t0 = clock64();
  int polls = 0;
  while (true) {
    __nanosleep(NS);
    if (mbar_try_wait_u32(addr, parity)) return true;
    if ((++polls & 63) == 0) {
      if (*ab.cta_flag != 0) return false;
      if (clock64() - t0 > kWaitBudgetCycles) {
        *ab.cta_flag = code;
        publish_abort(ab.global_status, code);
        return false;
      }
    }
  }
}
static __device__ __noinline__ bool mbar_wait_slow_u32(uint32_t bar, uint32_t parity, volatile int* cta_flag,
                                                       int* global_status, int code) {
  const long long t0 = clock64();
  int polls = 0;
  while (true) {
    if (mbar_try_wait_u32(bar, parity)) return true;
    if ((++polls & 63) == 0) {
      if (*cta_flag != 0) return false;
      if (clock64() - t0 > kWaitBudgetCycles) {
        *cta_flag = code;
        publish_abort(global_status, code);
        return false;
      }
    }
  }
}

// ---- TMA -----------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y,
                                            int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(z), "r"(w), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---- TMEM ----------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void tc_commit_u32(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 lanes x 32 columns: thread i of the warp receives columns [col, col+32) of TMEM lane
// (warp % 4) * 32 + i.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
      "%29,%30,%31}, [%32];"
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
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,"
      "%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
      "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
      "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(r[0]),
               "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}

// ---- UMMA descriptors ----------------------------------------------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle, version 1 (sm_100).  Addresses and byte
// offsets are stored without their 4 low bits.
//   K-major operand  (rows of 64 16-bit elements = 128 B): 8-row groups are sbo bytes apart.
//   MN-major operand (same tile used transposed): 64-element chunks along MN are lbo bytes
//   apart, groups of 8 along K are sbo bytes apart.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version
  d |= (uint64_t)2 << 61;  // SWIZZLE_128B
  return d;
}

// Instruction descriptor for kind::f16, fp32 accumulation.  fmt: 0 = f16, 1 = bf16.
__host__ __device__ constexpr uint32_t make_idesc(int fmt, int M, int N, int a_mn_major, int b_mn_major) {
  return (1u << 4) | ((uint32_t)fmt << 7) | ((uint32_t)fmt << 10) | ((uint32_t)a_mn_major << 15) |
         ((uint32_t)b_mn_major << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}


// The same two instructions with the shared-memory descriptors given as (low, high) words.  For the
// 128-byte-swizzled tiles used here (leading offset 16 B, 8-row groups 1024 B apart) the high word
// is the constant kDescHi and the low word is kDescLo | (byte address >> 4): stepping through a
// tile is an integer add on the low word.
constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
constexpr uint32_t kDescLo = (16u >> 4) << 16;
template <bool ACC>
__device__ __forceinline__ void umma_ss_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(kDescHi), "r"(idesc), "n"(ACC ? 1 : 0)
      : "memory");
}
template <bool ACC>
__device__ __forceinline__ void umma_ts_lo(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\tsetp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(kDescHi), "r"(idesc), "n"(ACC ? 1 : 0)
      : "memory");
}
// accumulate flag known only at run time
__device__ __forceinline__ void umma_ss_lo_dyn(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(kDescHi), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void umma_ts_lo_dyn(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\tsetp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(kDescHi), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Outputs of a launch that ran after a bounded wait gave up (or of the launch that gave up) are undefined.  To make
// that visible without a synchronisation, such a CTA stamps NaN into the statistics / leading elements of the rows
// it owns: every later reduction over the outputs, and every backward that reads lse, then carries NaN.
__device__ __forceinline__ float poison_f32() { return __uint_as_float(0x7fc00000u); }
template <typename T>
__device__ __forceinline__ void poison_row(void* base, size_t row, int D) {  // first 16 bytes of a (.., D) row
  uint4* p = reinterpret_cast<uint4*>(reinterpret_cast<T*>(base) + row * D);
  *p = sizeof(T) == 2 ? make_uint4(0x7fff7fffu, 0x7fff7fffu, 0x7fff7fffu, 0x7fff7fffu)
                      : make_uint4(0x7fc00000u, 0x7fc00000u, 0x7fc00000u, 0x7fc00000u);
}

template <int I>
struct IntC {
  static constexpr int value = I;
};

}  // namespace tc5
}  // namespace jvpfa
