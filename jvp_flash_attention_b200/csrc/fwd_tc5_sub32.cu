// Attention forward for head dimension 64 in 32-key sub-tiles (bf16 / fp16; none, causal, key
// padding) on tcgen05 / TMA / TMEM; dispatched for the primal-only forward (the kernel also handles
// tangents).  It is shaped by three measurements on B200:
//   * one thread issues a tcgen05.mma only about every 58-70 cycles whatever N <= 128 is;
//   * a hand-off through an mbarrier between two warps costs ~200 cycles, an
//     MMA -> tcgen05.commit -> waiting-thread hand-off ~300;
//   * the exponentials of a 64-key tile keep one warp's MUFU pipe busy for ~500 cycles.
// So the kernel keeps several things in flight per CTA instead of one strictly sequential chain:
//
//   - keys advance in sub-tiles of 32; the score accumulators [S | tS] (32 + 32 columns) exist twice,
//     so issuer A fills buffer (s+1)&1 while the softmax warps work on buffer s&1;
//   - two issuing warps with disjoint accumulator chains, and one N=64 / N=128 instruction wherever
//     two accumulators share the A operand and their B tiles are neighbours in shared memory:
//       issuer A:  [S | tS] = Q [K ; tK]^T  (N=64) ;  tS += tQ K^T  (N=32)        -> s_full[b]
//       issuer B:  [O | tO'] += P [V | tV]  (N=128) ;  tO' += W V    (N=64)       -> kv_empty[stage]
//   - P and W = P*tS*scale are written as packed 16-bit values over the head of S / tS of the same
//     buffer and are issuer B's TMEM A operands; issuer A reuses a buffer only after issuer B's
//     chain of the sub-tile two steps back has completed (kv_empty of that sub-tile's stage).
//
// CTA = one 128-row query tile of one (batch, head); 7 warps: TMA producer, issuer A, issuer B,
// four softmax / epilogue warps (thread <-> query row <-> TMEM lane).  TMEM (256 columns, two CTAs
// per SM):  buffer b at 64*b: S | tS ; O at 128 ; tO' at 192.
// Online softmax with lazy rescaling (O / tO' are touched only when the row maximum grows by more
// than 2^8, and then only after issuer B's previous chain has completed); packed fp32x2 arithmetic.
// Epilogue and saved statistics as in fwd_tc5.cu.
#include "tc5_common.cuh"

namespace jvpfa {
namespace tc5 {

template <bool DUAL>
struct FwdSub32Cfg {
  static constexpr int D = 64;
  static constexpr int BM = 128;
  static constexpr int BN = 32;
  static constexpr int STAGES = 4;
  static constexpr int NTHREADS = 224;
  static constexpr int Q_BYTES = BM * D * 2;   // 16 KiB
  static constexpr int KV_BYTES = BN * D * 2;  // 4 KiB
  static constexpr int N_Q = DUAL ? 2 : 1;
  static constexpr int N_KV = DUAL ? 4 : 2;
  // stage layout: K, tK, V, tV (DUAL) or K, V
  static constexpr int SLOT_K = 0, SLOT_TK = 1, SLOT_V = DUAL ? 2 : 1, SLOT_TV = 3;
  static constexpr int STAGE_BYTES = N_KV * KV_BYTES;
  static constexpr int TILE_BYTES = N_Q * Q_BYTES + STAGES * STAGE_BYTES;
  static constexpr int SMEM_BYTES = TILE_BYTES + 256 + 1024;
  static constexpr int COL_BUF = 64;  // columns per score buffer
  static constexpr int OFF_S = 0, OFF_TS = 32;
  static constexpr int COL_O = 128, COL_TO = 192;
  static constexpr int COLS_ALLOC = 256;
};

struct FwdSub32Maps {
  CUtensorMap q, tq, k, tk, v, tv;
};

__device__ __forceinline__ float2 fs2(uint32_t a, uint32_t b) { return make_float2(__uint_as_float(a), __uint_as_float(b)); }

template <typename T, bool DUAL>
__global__ void __launch_bounds__(224, 2)
fwd_tc5_sub32_kernel(const jvpfa_fwd_args a, const __grid_constant__ FwdSub32Maps maps, int* status) {
  using C = FwdSub32Cfg<DUAL>;
  constexpr int D = 64, BM = C::BM, BN = C::BN, STAGES = C::STAGES;

  if (*(volatile int*)status != 0) return;

  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  unsigned char* smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  unsigned char* sQ = smem;
  unsigned char* sTQ = sQ + C::Q_BYTES;  // DUAL only
  unsigned char* sKV = smem + C::N_Q * C::Q_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::TILE_BYTES);
  uint64_t* q_full = bars + 0;
  uint64_t* kv_full = bars + 1;            // [STAGES]
  uint64_t* kv_empty = bars + 1 + STAGES;  // [STAGES]
  uint64_t* s_full = bars + 1 + 2 * STAGES;  // [2]
  uint64_t* p_full = s_full + 2;             // [2]
  uint64_t* o_full = s_full + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_full + 5);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int L = a.L;
  const int bh = blockIdx.y;
  const int tma_b = bh / a.H, tma_h = bh - tma_b * a.H;  // coordinates in the (D, L, H, B) tensor maps
  const int b = bh / a.H;
  const int mt = (int)gridDim.x - 1 - (int)blockIdx.x;  // heaviest causal tiles first
  const int m0 = mt * BM;
  const bool causal = a.mask.kind == JVPFA_MASK_CAUSAL;
  int n_valid = L;
  if (a.mask.kind == JVPFA_MASK_KVLEN) {
    const int n = a.mask.kv_len[b];
    n_valid = n < 0 ? 0 : (n > L ? L : n);
  }
  int n_end = n_valid;
  if (causal) n_end = min(n_end, m0 + BM);
  const int n_sub = (n_end + BN - 1) / BN;

  if (tid == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(kv_full + s, 1);
      mbar_init(kv_empty + s, 1);
    }
    for (int g = 0; g < 2; ++g) {
      mbar_init(s_full + g, 1);
      mbar_init(p_full + g, 128);
    }
    mbar_init(o_full, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, C::COLS_ALLOC);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const AbortState ab{abort_flag, status};

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && n_sub > 0) {
      mbar_expect_tx(q_full, C::N_Q * C::Q_BYTES);
      tma_load_4d(sQ, &maps.q, q_full, 0, m0, tma_h, tma_b);
      if constexpr (DUAL) tma_load_4d(sTQ, &maps.tq, q_full, 0, m0, tma_h, tma_b);
      for (int s = 0; s < n_sub; ++s) {
        const int st = s % STAGES;
        const uint32_t ph = (s / STAGES) & 1;
        if (!mbar_wait(kv_empty + st, ph ^ 1, ab, kAbortKvEmpty)) break;
        unsigned char* base = sKV + st * C::STAGE_BYTES;
        mbar_expect_tx(kv_full + st, C::STAGE_BYTES);
        const int n0 = s * BN;
        tma_load_4d(base + C::SLOT_K * C::KV_BYTES, &maps.k, kv_full + st, 0, n0, tma_h, tma_b);
        tma_load_4d(base + C::SLOT_V * C::KV_BYTES, &maps.v, kv_full + st, 0, n0, tma_h, tma_b);
        if constexpr (DUAL) {
          tma_load_4d(base + C::SLOT_TK * C::KV_BYTES, &maps.tk, kv_full + st, 0, n0, tma_h, tma_b);
          tma_load_4d(base + C::SLOT_TV * C::KV_BYTES, &maps.tv, kv_full + st, 0, n0, tma_h, tma_b);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ issuer A: scores
    if (lane == 0 && n_sub > 0) {
      constexpr uint32_t idesc_s = make_idesc(Fmt<T>::kIdesc, BM, BN, 0, 0);       // 128 x 32
      constexpr uint32_t idesc_s2 = make_idesc(Fmt<T>::kIdesc, BM, 2 * BN, 0, 0);  // 128 x 64: [S | tS]
      const uint32_t aQ = smem_u32(sQ), aTQ = smem_u32(sTQ);
      bool ok = mbar_wait(q_full, 0, ab, kAbortQFull);
      for (int s = 0; ok && s < n_sub; ++s) {
        const int st = s % STAGES, buf = s & 1;
        // Buffer `buf` still holds P / W of sub-tile s-2 until issuer B's chain for it has completed.
        if (s >= 2 && !mbar_wait(kv_empty + ((s - 2) % STAGES), ((s - 2) / STAGES) & 1, ab, kAbortKvEmpty)) break;
        if (!mbar_wait(kv_full + st, (s / STAGES) & 1, ab, kAbortKvFull)) break;
        tc_fence_after();
        const uint32_t aK = smem_u32(sKV + st * C::STAGE_BYTES) + C::SLOT_K * C::KV_BYTES;
        const uint32_t dS = tmem + buf * C::COL_BUF + C::OFF_S;
        if constexpr (DUAL) {
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks)  // [S | tS] = Q [K ; tK]^T
            umma_ss(dS, make_smem_desc(aQ + ks * 32, 16, 1024), make_smem_desc(aK + ks * 32, 16, 1024), idesc_s2,
                    ks > 0);
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks)  // tS += tQ K^T
            umma_ss(tmem + buf * C::COL_BUF + C::OFF_TS, make_smem_desc(aTQ + ks * 32, 16, 1024),
                    make_smem_desc(aK + ks * 32, 16, 1024), idesc_s, 1);
        } else {
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks)
            umma_ss(dS, make_smem_desc(aQ + ks * 32, 16, 1024), make_smem_desc(aK + ks * 32, 16, 1024), idesc_s,
                    ks > 0);
        }
        tc_commit(s_full + buf);
      }
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------------ issuer B: outputs
    if (lane == 0 && n_sub > 0) {
      constexpr uint32_t idesc_o = make_idesc(Fmt<T>::kIdesc, BM, D, 0, 1);       // 128 x 64, B MN-major
      constexpr uint32_t idesc_o2 = make_idesc(Fmt<T>::kIdesc, BM, 2 * D, 0, 1);  // 128 x 128: [O | tO']
      for (int s = 0; s < n_sub; ++s) {
        const int st = s % STAGES, buf = s & 1;
        if (!mbar_wait(p_full + buf, (s >> 1) & 1, ab, kAbortPFull)) break;
        tc_fence_after();
        const uint32_t aV = smem_u32(sKV + st * C::STAGE_BYTES) + C::SLOT_V * C::KV_BYTES;
        const uint32_t tP = tmem + buf * C::COL_BUF + C::OFF_S, tW = tmem + buf * C::COL_BUF + C::OFF_TS;
        if constexpr (DUAL) {
#pragma unroll
          for (int kk = 0; kk < BN / 16; ++kk)  // [O | tO'] += P [V | tV]   (64-column chunks KV_BYTES apart)
            umma_ts(tmem + C::COL_O, tP + kk * 8, make_smem_desc(aV + kk * 2048, C::KV_BYTES, 1024), idesc_o2,
                    (s > 0 || kk > 0));
#pragma unroll
          for (int kk = 0; kk < BN / 16; ++kk)  // tO' += W V
            umma_ts(tmem + C::COL_TO, tW + kk * 8, make_smem_desc(aV + kk * 2048, C::KV_BYTES, 1024), idesc_o, 1);
        } else {
#pragma unroll
          for (int kk = 0; kk < BN / 16; ++kk)
            umma_ts(tmem + C::COL_O, tP + kk * 8, make_smem_desc(aV + kk * 2048, C::KV_BYTES, 1024), idesc_o,
                    (s > 0 || kk > 0));
        }
        tc_commit(kv_empty + st);
      }
      tc_commit(o_full);
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int i = m0 + row;
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t tbase = tmem + lane_off;
    const uint32_t tO = tbase + C::COL_O, tTO = tbase + C::COL_TO;
    const float scale_log2 = a.sm_scale * kLog2e;
    const float2 c2 = make_float2(scale_log2, scale_log2);
    const float2 sc2 = make_float2(a.sm_scale, a.sm_scale);
    float m_used = -INFINITY, l_run = 0.f, mu_run = 0.f;  // m_used: scaled (base-2) reference maximum
    bool alive = true;

    for (int s = 0; s < n_sub; ++s) {
      const int n0 = s * BN, buf = s & 1;
      const uint32_t tS = tbase + buf * C::COL_BUF + C::OFF_S, tTS = tbase + buf * C::COL_BUF + C::OFF_TS;
      if (!mbar_wait(s_full + buf, (s >> 1) & 1, ab, kAbortSFull)) {
        alive = false;
        break;
      }
      tc_fence_after();
      uint32_t x[32];
      uint32_t t[DUAL ? 32 : 1];
      tmem_ld32(tS, x);
      if constexpr (DUAL) tmem_ld32(tTS, t);
      tmem_wait_ld();
      // live key columns of this row inside the sub-tile: col < col_hi
      int col_hi = min(BN, n_valid - n0);
      if (causal) col_hi = min(col_hi, i - n0 + 1);
      const bool partial = (n0 + BN > n_valid) || (causal && n0 + BN - 1 > m0);
      if (partial) {
#pragma unroll
        for (int c = 0; c < 32; ++c)
          if (c >= col_hi) x[c] = 0xff800000u;  // -inf
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        mx0 = fmaxf(mx0, __uint_as_float(x[4 * c]));
        mx1 = fmaxf(mx1, __uint_as_float(x[4 * c + 1]));
        mx2 = fmaxf(mx2, __uint_as_float(x[4 * c + 2]));
        mx3 = fmaxf(mx3, __uint_as_float(x[4 * c + 3]));
      }
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * scale_log2;  // scale > 0 keeps the order
      // Lazy running max: keep the old reference while the new maximum is at most 2^8 above it.
      const bool grow = mx > m_used + 8.f;
      float alpha = 1.f;
      if (grow) {
        alpha = fast_exp2(m_used - mx);
        m_used = mx;
      }
      const float m_eff = (m_used == -INFINITY) ? 0.f : m_used;
      if (s > 0 && __any_sync(0xffffffffu, grow)) {
        // O / tO' may be rescaled only when issuer B's chain of the previous sub-tile has completed.
        if (!mbar_wait(kv_empty + ((s - 1) % STAGES), ((s - 1) / STAGES) & 1, ab, kAbortKvEmpty)) {
          alive = false;
          break;
        }
        tc_fence_after();
        const float2 al2 = make_float2(alpha, alpha);
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(tO + 32 * c, r);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const float2 v = __fmul2_rn(fs2(r[2 * e], r[2 * e + 1]), al2);
            r[2 * e] = __float_as_uint(v.x), r[2 * e + 1] = __float_as_uint(v.y);
          }
          tmem_st32(tO + 32 * c, r);
          if constexpr (DUAL) {
            tmem_ld32(tTO + 32 * c, r);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              const float2 v = __fmul2_rn(fs2(r[2 * e], r[2 * e + 1]), al2);
              r[2 * e] = __float_as_uint(v.x), r[2 * e + 1] = __float_as_uint(v.y);
            }
            tmem_st32(tTO + 32 * c, r);
          }
        }
      }
      const float2 nm2 = make_float2(-m_eff, -m_eff);
      float2 ls2a = make_float2(0.f, 0.f), ls2b = make_float2(0.f, 0.f);
      float2 ms2a = make_float2(0.f, 0.f), ms2b = make_float2(0.f, 0.f);
      uint32_t pp[16];
      uint32_t wp[DUAL ? 16 : 1];
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        const float2 e = __ffma2_rn(fs2(x[2 * c], x[2 * c + 1]), c2, nm2);  // masked: -inf*c - m = -inf
        const float2 p = make_float2(fast_exp2(e.x), fast_exp2(e.y));
        if (c & 1) ls2b = __fadd2_rn(ls2b, p);
        else ls2a = __fadd2_rn(ls2a, p);
        pp[c] = Elem<T>::pack(p.x, p.y);
        if constexpr (DUAL) {
          const float2 w = __fmul2_rn(p, __fmul2_rn(fs2(t[2 * c], t[2 * c + 1]), sc2));
          if (c & 1) ms2b = __fadd2_rn(ms2b, w);
          else ms2a = __fadd2_rn(ms2a, w);
          wp[c] = Elem<T>::pack(w.x, w.y);
        }
      }
      l_run = l_run * alpha + ((ls2a.x + ls2a.y) + (ls2b.x + ls2b.y));
      if constexpr (DUAL) mu_run = mu_run * alpha + ((ms2a.x + ms2a.y) + (ms2b.x + ms2b.y));
      tmem_st16(tS, pp);
      if constexpr (DUAL) tmem_st16(tTS, wp);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(p_full + buf);
    }

    // ---- epilogue ----
    if (alive && n_sub > 0) alive = mbar_wait(o_full, 0, ab, kAbortOFull);
    if (alive) {
      tc_fence_after();
      const bool empty = !(l_run > 0.f);
      const float inv_l = empty ? 0.f : 1.f / l_run;
      const float mu_n = mu_run * inv_l;
      const bool in_range = i < L;
      if (in_range) {
        a.lse[(size_t)bh * L + i] = empty ? INFINITY : (m_used + log2f(l_run));
        if constexpr (DUAL) a.mu[(size_t)bh * L + i] = mu_n;
      }
      T* gO = reinterpret_cast<T*>(a.o) + ((size_t)bh * L + i) * D;
      T* gTO = DUAL ? reinterpret_cast<T*>(a.to) + ((size_t)bh * L + i) * D : nullptr;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t ro[32];
        uint32_t po[16];
        if (n_sub > 0) {
          tmem_ld32(tO + 32 * c, ro);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) ro[e] = 0u;
        }
#pragma unroll
        for (int e = 0; e < 32; ++e) ro[e] = __float_as_uint(__uint_as_float(ro[e]) * inv_l);
#pragma unroll
        for (int e = 0; e < 16; ++e) po[e] = Elem<T>::pack(__uint_as_float(ro[2 * e]), __uint_as_float(ro[2 * e + 1]));
        if (in_range) {
#pragma unroll
          for (int e = 0; e < 4; ++e)
            reinterpret_cast<uint4*>(gO + 32 * c)[e] = make_uint4(po[4 * e], po[4 * e + 1], po[4 * e + 2], po[4 * e + 3]);
        }
        if constexpr (DUAL) {
          uint32_t rt[32];
          if (n_sub > 0) {
            tmem_ld32(tTO + 32 * c, rt);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) rt[e] = 0u;
          }
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const float t0 = __uint_as_float(rt[2 * e]) * inv_l - mu_n * __uint_as_float(ro[2 * e]);
            const float t1 = __uint_as_float(rt[2 * e + 1]) * inv_l - mu_n * __uint_as_float(ro[2 * e + 1]);
            po[e] = Elem<T>::pack(t0, t1);
          }
          if (in_range) {
#pragma unroll
            for (int e = 0; e < 4; ++e)
              reinterpret_cast<uint4*>(gTO + 32 * c)[e] =
                  make_uint4(po[4 * e], po[4 * e + 1], po[4 * e + 2], po[4 * e + 3]);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    if (*abort_flag != 0) {
      const long long t0 = clock64();
      while (clock64() - t0 < (1ll << 22)) {
      }
    }
    tc_fence_after();
    tmem_dealloc(tmem, C::COLS_ALLOC);
  }
}

template <typename T, bool DUAL>
static int launch_fwd_sub32(const jvpfa_fwd_args& a, cudaStream_t stream) {
  using C = FwdSub32Cfg<DUAL>;
  int* status = tc5_status_device_ptr();
  if (!status) {
    set_last_cuda_error(cudaErrorUnknown, "status word address");
    return JVPFA_ERR_CUDA;
  }
  FwdSub32Maps maps;
  const long long BH = (long long)a.B * a.H;
  const CUtensorMapDataType dt = Fmt<T>::kTma;
  bool ok = encode_map4d(&maps.q, dt, a.q, 64, a.L, a.H, a.B, a.in_stride, C::BM) && encode_map4d(&maps.k, dt, a.k, 64, a.L, a.H, a.B, a.in_stride, C::BN) &&
            encode_map4d(&maps.v, dt, a.v, 64, a.L, a.H, a.B, a.in_stride, C::BN);
  if (DUAL)
    ok = ok && encode_map4d(&maps.tq, dt, a.tq, 64, a.L, a.H, a.B, a.in_stride, C::BM) && encode_map4d(&maps.tk, dt, a.tk, 64, a.L, a.H, a.B, a.in_stride, C::BN) &&
         encode_map4d(&maps.tv, dt, a.tv, 64, a.L, a.H, a.B, a.in_stride, C::BN);
  else
    maps.tq = maps.tk = maps.tv = maps.q;
  if (!ok) {
    set_last_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled(fwd d64)");
    return JVPFA_ERR_CUDA;
  }
  auto kern = fwd_tc5_sub32_kernel<T, DUAL>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
  if (e != cudaSuccess) {
    set_last_cuda_error(e, "cudaFuncSetAttribute(fwd_tc5_d64)");
    return JVPFA_ERR_CUDA;
  }
  dim3 grid((a.L + C::BM - 1) / C::BM, a.B * a.H);
  kern<<<grid, C::NTHREADS, C::SMEM_BYTES, stream>>>(a, maps, status);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_cuda_error(e, "launch fwd_tc5_d64");
    return JVPFA_ERR_CUDA;
  }
  return JVPFA_OK;
}

}  // namespace tc5

// Used for the primal-only forward.  (With tangents the score MMAs would take Q and tQ from shared
// memory once per 32-key sub-tile; measured, that re-reading makes the 64-key variant in
// fwd_tc5_d64.cu the faster one, 0.19 ms against 0.21 ms on B4 H16 L2048 causal.)
int launch_fwd_tc5_sub32(const jvpfa_fwd_args& a, cudaStream_t s) {
  const bool dual = a.tq != nullptr;
  if (a.dtype == JVPFA_BF16)
    return dual ? tc5::launch_fwd_sub32<__nv_bfloat16, true>(a, s) : tc5::launch_fwd_sub32<__nv_bfloat16, false>(a, s);
  return dual ? tc5::launch_fwd_sub32<__half, true>(a, s) : tc5::launch_fwd_sub32<__half, false>(a, s);
}

}  // namespace jvpfa
