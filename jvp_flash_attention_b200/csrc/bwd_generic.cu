// Backward of  <gO, O> + <gtO, tO>  with respect to q, k, v on warp-level tensor-core MMAs.
//
// Per head, with s = sm_scale, S = s Q K^T + bias, P = softmax(S), tS = s (tQ K^T + Q tK^T),
// mu = rowsum(P*tS), O = P V, tO = (P*(tS - mu)) V + P tV, and cotangents gO, G = gtO:
//
//   delta = rowsum(gO*O)   eps = rowsum(G*O)   cterm = rowsum(G*tO) - eps*mu     (preprocess)
//   dP = gO V^T   E = G V^T   F = G tV^T
//   gtS = P*(E - eps)
//   gS  = P*( E*(tS - mu) - eps*tS + F + dP - delta - cterm )
//   dV = P^T gO + (P*(tS - mu))^T G
//   dQ = s (gS K + gtS tK)          dK = s (gS^T Q + gtS^T tQ)
//
// With G absent this reduces to the flash-attention-2 backward that upstream implements in
// _attn_bwd_dkdv / _attn_bwd_dq (jvp_flash_attention/jvp_attention.py:1415-1707).  Like upstream
// (jvp_attention.py:2008-2233) the work is split into a kernel that owns a key tile and loops
// over query tiles (dK, dV) and one that owns a query tile and loops over key tiles (dQ); score
// tiles are recomputed from the saved base-2 logsumexp, so results are deterministic and no
// L x L tensor or atomic accumulation is needed.
#include "common.cuh"

namespace jvpfa {

// ----------------------------------------------------------------------------------------------
// Preprocess: three row reductions, one pass over O, tO, gO, gtO (HBM bound).
// ----------------------------------------------------------------------------------------------
template <typename T>
struct Vec16 {
  static constexpr int N = 16 / (int)sizeof(T);
  T v[N];
};

template <typename T, int D>
__global__ void __launch_bounds__(256) pre_kernel(const jvpfa_pre_args a, long long rows) {
  constexpr int VEC = 16 / (int)sizeof(T);
  constexpr int TPR = D / VEC;  // threads per row (4..32)
  constexpr int RPB = 256 / TPR;
  const int tid = threadIdx.x;
  const long long row = (long long)blockIdx.x * RPB + tid / TPR;
  const int c = (tid % TPR) * VEC;
  const bool ok = row < rows;
  const bool has_go = a.go != nullptr, has_g = a.gto != nullptr;

  float d = 0.f, e = 0.f, dd = 0.f;
  if (ok) {
    const size_t off = (size_t)row * D + c;
    uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(a.o) + off);
    const Vec16<T>& vo = *reinterpret_cast<const Vec16<T>*>(&raw);
    if (has_go) {
      uint4 r2 = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(a.go) + off);
      const Vec16<T>& vg = *reinterpret_cast<const Vec16<T>*>(&r2);
#pragma unroll
      for (int i = 0; i < VEC; ++i) d += Elem<T>::to_float(vo.v[i]) * Elem<T>::to_float(vg.v[i]);
    }
    if (has_g) {
      uint4 r3 = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(a.gto) + off);
      uint4 r4 = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(a.to) + off);
      const Vec16<T>& vg = *reinterpret_cast<const Vec16<T>*>(&r3);
      const Vec16<T>& vt = *reinterpret_cast<const Vec16<T>*>(&r4);
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        const float gg = Elem<T>::to_float(vg.v[i]);
        e += gg * Elem<T>::to_float(vo.v[i]);
        dd += gg * Elem<T>::to_float(vt.v[i]);
      }
    }
  }
#pragma unroll
  for (int o = TPR / 2; o > 0; o >>= 1) {
    d += __shfl_xor_sync(0xffffffffu, d, o);
    e += __shfl_xor_sync(0xffffffffu, e, o);
    dd += __shfl_xor_sync(0xffffffffu, dd, o);
  }
  if (ok && (tid % TPR) == 0) {
    a.delta[row] = d;
    a.eps[row] = e;
    a.cterm[row] = has_g ? dd - e * a.mu[row] : 0.f;
  }
}

template <typename T, int D>
static int launch_pre_one(const jvpfa_pre_args& a, cudaStream_t stream) {
  constexpr int VEC = 16 / (int)sizeof(T);
  constexpr int RPB = 256 / (D / VEC);
  const long long rows = (long long)a.B * a.H * a.L;
  const long long blocks = (rows + RPB - 1) / RPB;
  pre_kernel<T, D><<<(unsigned)blocks, 256, 0, stream>>>(a, rows);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_cuda_error(e, "launch pre_kernel");
    return JVPFA_ERR_CUDA;
  }
  return JVPFA_OK;
}

template <typename T>
static int launch_pre_t(const jvpfa_pre_args& a, cudaStream_t s) {
  switch (a.D) {
    case 32:
      return launch_pre_one<T, 32>(a, s);
    case 64:
      return launch_pre_one<T, 64>(a, s);
    case 128:
      return launch_pre_one<T, 128>(a, s);
    default:
      return JVPFA_ERR_SHAPE;
  }
}

int launch_pre(const jvpfa_pre_args& a, cudaStream_t s) {
  switch (a.dtype) {
    case JVPFA_BF16:
      return launch_pre_t<__nv_bfloat16>(a, s);
    case JVPFA_FP16:
      return launch_pre_t<__half>(a, s);
    case JVPFA_FP32:
    case JVPFA_FP32_TF32:  // no products in this kernel
      return launch_pre_t<float>(a, s);
    default:
      return JVPFA_ERR_DTYPE;
  }
}

// ----------------------------------------------------------------------------------------------
// Main kernels
// ----------------------------------------------------------------------------------------------
template <typename T, int D>
struct BwdCfg {
  static constexpr int OWN = 64;  // rows owned by the CTA (4 warps x 16)
  static constexpr int LOOP = (Elem<T>::k16 && D <= 64) ? 64 : 32;
  static constexpr int LD = D + Elem<T>::kPad;
  static constexpr int NTHREADS = 128;
  static constexpr int STAGES = (!Elem<T>::k16 && D >= 128) ? 1 : 2;
  static constexpr int NSTAT = 5;  // lse, delta, eps, cterm, mu
  // own_tiles / loop_tiles = number of [rows][D] operand tiles of each kind
  static constexpr size_t smem(int own_tiles, int loop_tiles, bool stats) {
    return sizeof(T) * ((size_t)own_tiles * OWN * LD + (size_t)STAGES * loop_tiles * LOOP * LD) +
           (stats ? sizeof(float) * STAGES * NSTAT * LOOP : 0);
  }
};

template <int N>
__device__ __forceinline__ void zero_acc(float (*x)[4]) {
#pragma unroll
  for (int i = 0; i < N; ++i) {
    x[i][0] = 0.f;
    x[i][1] = 0.f;
    x[i][2] = 0.f;
    x[i][3] = 0.f;
  }
}

// acc[NTILES][4] += A[r0..r0+15][0..D) * B[0..8*NTILES)[0..D)^T   (both operands D-contiguous)
template <typename T, int D, int NTILES>
__device__ __forceinline__ void gemm_nt(float (*acc)[4], const T* sA, const T* sB, int ld, int r0, int lane) {
  constexpr int KS = Elem<T>::kKStep;
#pragma unroll
  for (int k0 = 0; k0 < D; k0 += KS) {
    FragA<T> fa;
    load_a<T>(fa, sA, ld, r0, k0, lane);
#pragma unroll
    for (int nt = 0; nt < NTILES; ++nt) {
      FragB<T> fb;
      load_b_nt<T>(fb, sB, ld, nt * 8, k0, lane);
      mma<T>(acc[nt], fa, fb);
    }
  }
}

// out[D/8][4] += Atile(accumulator layout, 16 x KROWS) * B[0..KROWS)[0..D)   (B is [k][d], d contiguous)
template <typename T, int D, int KROWS>
__device__ __forceinline__ void gemm_acc_nn(float (*out)[4], const float (*atile)[4], const T* sB, int ld,
                                            int lane) {
  constexpr int KS = Elem<T>::kKStep;
  if constexpr (Elem<T>::k16) {
#pragma unroll
    for (int kk = 0; kk < KROWS / KS; ++kk) {
      FragA<T> fa;
      a_from_acc<T>(fa, atile, kk);
#pragma unroll
      for (int dt = 0; dt < D / 8; ++dt) {
        FragB<T> fb;
        load_b_nn<T>(fb, sB, ld, kk * KS, dt * 8, lane);
        mma<T>(out[dt], fa, fb);
      }
    }
  } else {
    // fp32: the tensor core adds into its fp32 accumulator with truncation, and hundreds of such
    // adds into one long-lived accumulator show up as a bias of ~1e-5.  Accumulate this tile's
    // contribution in a fresh register tile (32 columns at a time) and add it once, rounded.
#pragma unroll
    for (int d0 = 0; d0 < D / 8; d0 += 4) {
      float tmp[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) tmp[i][0] = tmp[i][1] = tmp[i][2] = tmp[i][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < KROWS / KS; ++kk) {
        FragA<T> fa;
        a_from_acc<T>(fa, atile, kk);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          FragB<T> fb;
          load_b_nn<T>(fb, sB, ld, kk * KS, (d0 + i) * 8, lane);
          mma<T>(tmp[i], fa, fb);
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        out[d0 + i][0] += tmp[i][0];
        out[d0 + i][1] += tmp[i][1];
        out[d0 + i][2] += tmp[i][2];
        out[d0 + i][3] += tmp[i][3];
      }
    }
  }
}

// Writes a warp's 16 x D accumulator strip (scaled) into a padded smem tile as T.
template <typename T, int D>
__device__ __forceinline__ void acc_to_smem(T* s, int ld, int r0, int lane, const float (*acc)[4], float scale) {
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int dt = 0; dt < D / 8; ++dt) {
    T* lo = s + (r0 + g) * ld + dt * 8 + 2 * t;
    T* hi = lo + 8 * ld;
    lo[0] = Elem<T>::from_float(acc[dt][0] * scale);
    lo[1] = Elem<T>::from_float(acc[dt][1] * scale);
    hi[0] = Elem<T>::from_float(acc[dt][2] * scale);
    hi[1] = Elem<T>::from_float(acc[dt][3] * scale);
  }
}

template <typename T, int ROWS, int D, int NTHREADS>
__device__ __forceinline__ void smem_tile_to_global(T* ghead, const T* s, int ld, int row0, int L, int tid) {
  constexpr int VEC = 16 / (int)sizeof(T);
  constexpr int VPR = D / VEC;
  for (int idx = tid; idx < ROWS * VPR; idx += NTHREADS) {
    const int r = idx / VPR, c = (idx - r * VPR) * VEC;
    const int row = row0 + r;
    if (row < L)
      *reinterpret_cast<uint4*>(ghead + (size_t)row * D + c) = *reinterpret_cast<const uint4*>(s + r * ld + c);
  }
}

// ---- dK, dV: CTA owns 64 keys, loops over query tiles.  Tiles are held transposed
// (rows = keys, columns = queries) so that P^T etc. feed the second MMAs from registers. ----
template <typename T, int D, bool HAS_GO, bool HAS_GT>
__global__ void __launch_bounds__(128) bwd_dkdv_kernel(const jvpfa_bwd_args a) {
  using C = BwdCfg<T, D>;
  constexpr int BN = C::OWN, BM = C::LOOP, LD = C::LD, NT = C::NTHREADS, STAGES = C::STAGES;
  constexpr int NQ = BM / 8;
  constexpr int ND = D / 8;
  constexpr int OWN_TILES = HAS_GT ? 4 : 2;
  constexpr int LOOP_TILES = 1 + (HAS_GO ? 1 : 0) + (HAS_GT ? 2 : 0);

  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* sK = reinterpret_cast<T*>(smem_raw);
  T* sV = sK + BN * LD;
  T* sTK = sK + 2 * BN * LD;  // HAS_GT only
  T* sTV = sK + 3 * BN * LD;  // HAS_GT only
  T* sLoop = sK + OWN_TILES * BN * LD;
  float* sStat = reinterpret_cast<float*>(sLoop + (size_t)STAGES * LOOP_TILES * BM * LD);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int L = a.L;
  const int bh = blockIdx.y;
  const int b = bh / a.H, h = bh - b * a.H;
  const int n0 = blockIdx.x * BN;
  const size_t head_off = (size_t)bh * L * D;
  const size_t stat_off = (size_t)bh * L;

  // the six inputs may share a strided (batch, head, row) layout (in_stride, elements; all zero = row-major)
  const bool strided = (a.in_stride[0] | a.in_stride[1] | a.in_stride[2]) != 0;
  const long long in_off = strided ? (long long)b * a.in_stride[0] + (long long)h * a.in_stride[1] : (long long)head_off;
  const long long in_rs = strided ? a.in_stride[2] : D;
  const T* gQ = reinterpret_cast<const T*>(a.q) + in_off;
  const T* gK = reinterpret_cast<const T*>(a.k) + in_off;
  const T* gV = reinterpret_cast<const T*>(a.v) + in_off;
  const T* gTQ = HAS_GT ? reinterpret_cast<const T*>(a.tq) + in_off : nullptr;
  const T* gTK = HAS_GT ? reinterpret_cast<const T*>(a.tk) + in_off : nullptr;
  const T* gTV = HAS_GT ? reinterpret_cast<const T*>(a.tv) + in_off : nullptr;
  const T* gGO = HAS_GO ? reinterpret_cast<const T*>(a.go) + head_off : nullptr;
  const T* gG = HAS_GT ? reinterpret_cast<const T*>(a.gto) + head_off : nullptr;

  const MaskView mv = make_mask_view(a.mask, b, h, L);

  // Query tiles that can see this key tile.
  int m_begin = 0;
  if (mv.kind == JVPFA_MASK_CAUSAL) m_begin = (n0 / BM) * BM;
  int n_tiles = (L - m_begin + BM - 1) / BM;
  if (mv.kind == JVPFA_MASK_KVLEN && n0 >= mv.kv_len) n_tiles = 0;

  auto stage_loop = [&](int stage, int m0) {
    T* base = sLoop + (size_t)stage * LOOP_TILES * BM * LD;
    int k = 0;
    stage_tile<T, BM, D, NT>(base + (k++) * BM * LD, gQ, m0, L, tid, in_rs);
    if constexpr (HAS_GO) stage_tile<T, BM, D, NT>(base + (k++) * BM * LD, gGO, m0, L, tid);
    if constexpr (HAS_GT) {
      stage_tile<T, BM, D, NT>(base + (k++) * BM * LD, gTQ, m0, L, tid, in_rs);
      stage_tile<T, BM, D, NT>(base + (k++) * BM * LD, gG, m0, L, tid);
    }
    if (tid < BM) {
      float* st = sStat + stage * C::NSTAT * BM;
      const int i = m0 + tid;
      const bool ok = i < L;
      st[0 * BM + tid] = ok ? a.lse[stat_off + i] : INFINITY;
      st[1 * BM + tid] = ok ? a.delta[stat_off + i] : 0.f;
      if constexpr (HAS_GT) {
        st[2 * BM + tid] = ok ? a.eps[stat_off + i] : 0.f;
        st[3 * BM + tid] = ok ? a.cterm[stat_off + i] : 0.f;
        st[4 * BM + tid] = ok ? a.mu[stat_off + i] : 0.f;
      }
    }
  };

  stage_tile<T, BN, D, NT>(sK, gK, n0, L, tid, in_rs);
  stage_tile<T, BN, D, NT>(sV, gV, n0, L, tid, in_rs);
  if constexpr (HAS_GT) {
    stage_tile<T, BN, D, NT>(sTK, gTK, n0, L, tid, in_rs);
    stage_tile<T, BN, D, NT>(sTV, gTV, n0, L, tid, in_rs);
  }
  if (STAGES == 2 && n_tiles > 0) stage_loop(0, m_begin);
  cp_async_commit();

  const float scale_log2 = a.sm_scale * kLog2e;
  const int r0 = warp * 16;
  const int key_lo = n0 + r0 + g, key_hi = key_lo + 8;

  float dk[ND][4], dv[ND][4];
  zero_acc<ND>(dk);
  zero_acc<ND>(dv);

  for (int it = 0; it < n_tiles; ++it) {
    const int m0 = m_begin + it * BM;
    int stage;
    if (STAGES == 2) {
      if (it + 1 < n_tiles) stage_loop((it + 1) & 1, m0 + BM);
      cp_async_commit();
      cp_async_wait<1>();
      stage = it & 1;
    } else {
      stage_loop(0, m0);
      cp_async_commit();
      cp_async_wait<0>();
      stage = 0;
    }
    __syncthreads();

    const T* base = sLoop + (size_t)stage * LOOP_TILES * BM * LD;
    const T* sQ = base;
    const T* sGO = base + BM * LD;                       // HAS_GO
    const T* sTQ = base + (1 + (HAS_GO ? 1 : 0)) * BM * LD;  // HAS_GT
    const T* sG = sTQ + BM * LD;                          // HAS_GT
    const float* st = sStat + stage * C::NSTAT * BM;

    // P^T
    float p[NQ][4];
    zero_acc<NQ>(p);
    gemm_nt<T, D, NQ>(p, sK, sQ, LD, r0, lane);
#pragma unroll
    for (int nt = 0; nt < NQ; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = (e < 2) ? key_lo : key_hi;
        const int ci = nt * 8 + 2 * t + (e & 1);
        const int i = m0 + ci;
        float v = 0.f;
        if (mv.allowed(i, j)) {
          const float x = p[nt][e] * scale_log2 + mv.bias(i, j) * kLog2e;
          v = exp2f(x - st[ci]);
        }
        p[nt][e] = v;
      }
    }
    if constexpr (HAS_GO) gemm_acc_nn<T, D, BM>(dv, p, sGO, LD, lane);

    float acc[NQ][4];
    zero_acc<NQ>(acc);
    if constexpr (HAS_GT) {
      float ts[NQ][4];
      zero_acc<NQ>(ts);
      gemm_nt<T, D, NQ>(ts, sK, sTQ, LD, r0, lane);
      gemm_nt<T, D, NQ>(ts, sTK, sQ, LD, r0, lane);
      gemm_nt<T, D, NQ>(acc, sV, sG, LD, r0, lane);  // E^T
      {
        float w[NQ][4];
#pragma unroll
        for (int nt = 0; nt < NQ; ++nt) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int ci = nt * 8 + 2 * t + (e & 1);
            ts[nt][e] *= a.sm_scale;
            w[nt][e] = p[nt][e] * (ts[nt][e] - st[4 * BM + ci]);
          }
        }
        gemm_acc_nn<T, D, BM>(dv, w, sG, LD, lane);  // (P*(tS-mu))^T G
#pragma unroll
        for (int nt = 0; nt < NQ; ++nt) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int ci = nt * 8 + 2 * t + (e & 1);
            w[nt][e] = p[nt][e] * (acc[nt][e] - st[2 * BM + ci]);
          }
        }
        gemm_acc_nn<T, D, BM>(dk, w, sTQ, LD, lane);  // gtS^T tQ
      }
#pragma unroll
      for (int nt = 0; nt < NQ; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int ci = nt * 8 + 2 * t + (e & 1);
          const float tsv = ts[nt][e];
          acc[nt][e] = acc[nt][e] * (tsv - st[4 * BM + ci]) - st[2 * BM + ci] * tsv;
        }
      }
      gemm_nt<T, D, NQ>(acc, sTV, sG, LD, r0, lane);  // + F^T
    }
    if constexpr (HAS_GO) gemm_nt<T, D, NQ>(acc, sV, sGO, LD, r0, lane);  // + dP^T
#pragma unroll
    for (int nt = 0; nt < NQ; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int ci = nt * 8 + 2 * t + (e & 1);
        float sub = st[1 * BM + ci];
        if constexpr (HAS_GT) sub += st[3 * BM + ci];
        acc[nt][e] = p[nt][e] * (acc[nt][e] - sub);
      }
    }
    gemm_acc_nn<T, D, BM>(dk, acc, sQ, LD, lane);  // gS^T Q
    __syncthreads();
  }
  cp_async_wait<0>();
  __syncthreads();

  // Own K / V buffers are idle now: reuse them to coalesce the stores.
  acc_to_smem<T, D>(sK, LD, r0, lane, dk, a.sm_scale);
  acc_to_smem<T, D>(sV, LD, r0, lane, dv, 1.f);
  __syncthreads();
  smem_tile_to_global<T, BN, D, NT>(reinterpret_cast<T*>(a.dk) + head_off, sK, LD, n0, L, tid);
  smem_tile_to_global<T, BN, D, NT>(reinterpret_cast<T*>(a.dv) + head_off, sV, LD, n0, L, tid);
}

// ---- dQ: CTA owns 64 queries, loops over key tiles (rows = queries, columns = keys). ----
template <typename T, int D, bool HAS_GO, bool HAS_GT>
__global__ void __launch_bounds__(128) bwd_dq_kernel(const jvpfa_bwd_args a) {
  using C = BwdCfg<T, D>;
  constexpr int BM = C::OWN, BN = C::LOOP, LD = C::LD, NT = C::NTHREADS, STAGES = C::STAGES;
  constexpr int NK = BN / 8;
  constexpr int ND = D / 8;
  constexpr int OWN_TILES = 1 + (HAS_GO ? 1 : 0) + (HAS_GT ? 2 : 0);
  constexpr int LOOP_TILES = HAS_GT ? 4 : 2;

  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* sQ = reinterpret_cast<T*>(smem_raw);
  T* sGO = sQ + BM * LD;                              // HAS_GO
  T* sTQ = sQ + (1 + (HAS_GO ? 1 : 0)) * BM * LD;     // HAS_GT
  T* sG = sTQ + BM * LD;                              // HAS_GT
  T* sLoop = sQ + OWN_TILES * BM * LD;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int L = a.L;
  const int bh = blockIdx.y;
  const int b = bh / a.H, h = bh - b * a.H;
  const int mt = (int)gridDim.x - 1 - (int)blockIdx.x;
  const int m0 = mt * BM;
  const size_t head_off = (size_t)bh * L * D;
  const size_t stat_off = (size_t)bh * L;

  // the six inputs may share a strided (batch, head, row) layout (in_stride, elements; all zero = row-major)
  const bool strided = (a.in_stride[0] | a.in_stride[1] | a.in_stride[2]) != 0;
  const long long in_off = strided ? (long long)b * a.in_stride[0] + (long long)h * a.in_stride[1] : (long long)head_off;
  const long long in_rs = strided ? a.in_stride[2] : D;
  const T* gQ = reinterpret_cast<const T*>(a.q) + in_off;
  const T* gK = reinterpret_cast<const T*>(a.k) + in_off;
  const T* gV = reinterpret_cast<const T*>(a.v) + in_off;
  const T* gTQ = HAS_GT ? reinterpret_cast<const T*>(a.tq) + in_off : nullptr;
  const T* gTK = HAS_GT ? reinterpret_cast<const T*>(a.tk) + in_off : nullptr;
  const T* gTV = HAS_GT ? reinterpret_cast<const T*>(a.tv) + in_off : nullptr;
  const T* gGO = HAS_GO ? reinterpret_cast<const T*>(a.go) + head_off : nullptr;
  const T* gG = HAS_GT ? reinterpret_cast<const T*>(a.gto) + head_off : nullptr;

  const MaskView mv = make_mask_view(a.mask, b, h, L);

  int n_end = L;
  if (mv.kind == JVPFA_MASK_CAUSAL) n_end = min(L, m0 + BM);
  if (mv.kind == JVPFA_MASK_KVLEN) n_end = min(L, mv.kv_len);
  const int n_tiles = (n_end + BN - 1) / BN;

  auto stage_loop = [&](int stage, int n0) {
    T* base = sLoop + (size_t)stage * LOOP_TILES * BN * LD;
    stage_tile<T, BN, D, NT>(base, gK, n0, L, tid, in_rs);
    stage_tile<T, BN, D, NT>(base + BN * LD, gV, n0, L, tid, in_rs);
    if constexpr (HAS_GT) {
      stage_tile<T, BN, D, NT>(base + 2 * BN * LD, gTK, n0, L, tid, in_rs);
      stage_tile<T, BN, D, NT>(base + 3 * BN * LD, gTV, n0, L, tid, in_rs);
    }
  };

  stage_tile<T, BM, D, NT>(sQ, gQ, m0, L, tid, in_rs);
  if constexpr (HAS_GO) stage_tile<T, BM, D, NT>(sGO, gGO, m0, L, tid);
  if constexpr (HAS_GT) {
    stage_tile<T, BM, D, NT>(sTQ, gTQ, m0, L, tid, in_rs);
    stage_tile<T, BM, D, NT>(sG, gG, m0, L, tid);
  }
  if (STAGES == 2 && n_tiles > 0) stage_loop(0, 0);
  cp_async_commit();

  const float scale_log2 = a.sm_scale * kLog2e;
  const int r0 = warp * 16;
  const int row[2] = {m0 + r0 + g, m0 + r0 + g + 8};
  float lse[2], sub[2], eps[2] = {0.f, 0.f}, mu[2] = {0.f, 0.f};
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const bool ok = row[r] < L;
    lse[r] = ok ? a.lse[stat_off + row[r]] : INFINITY;
    sub[r] = ok ? a.delta[stat_off + row[r]] : 0.f;
    if constexpr (HAS_GT) {
      sub[r] += ok ? a.cterm[stat_off + row[r]] : 0.f;
      eps[r] = ok ? a.eps[stat_off + row[r]] : 0.f;
      mu[r] = ok ? a.mu[stat_off + row[r]] : 0.f;
    }
  }

  float dq[ND][4];
  zero_acc<ND>(dq);

  for (int it = 0; it < n_tiles; ++it) {
    const int n0 = it * BN;
    int stage;
    if (STAGES == 2) {
      if (it + 1 < n_tiles) stage_loop((it + 1) & 1, n0 + BN);
      cp_async_commit();
      cp_async_wait<1>();
      stage = it & 1;
    } else {
      stage_loop(0, n0);
      cp_async_commit();
      cp_async_wait<0>();
      stage = 0;
    }
    __syncthreads();

    const T* sK = sLoop + (size_t)stage * LOOP_TILES * BN * LD;
    const T* sV = sK + BN * LD;
    const T* sTK = sK + 2 * BN * LD;
    const T* sTV = sK + 3 * BN * LD;

    float p[NK][4];
    zero_acc<NK>(p);
    gemm_nt<T, D, NK>(p, sQ, sK, LD, r0, lane);
#pragma unroll
    for (int nt = 0; nt < NK; ++nt) {
#pragma unroll
      for (int r = 0; r < 2; ++r) {  // accumulator elements 2r, 2r+1: one query row, keys j and j + 1
        bool ok[2];
        float bias[2];
        mv.pair(row[r], n0 + nt * 8 + 2 * t, ok, bias);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int e = 2 * r + c;
          float v = 0.f;
          if (ok[c]) v = exp2f(p[nt][e] * scale_log2 + bias[c] * kLog2e - lse[r]);
          p[nt][e] = v;
        }
      }
    }

    float acc[NK][4];
    zero_acc<NK>(acc);
    if constexpr (HAS_GT) {
      float ts[NK][4];
      zero_acc<NK>(ts);
      gemm_nt<T, D, NK>(ts, sTQ, sK, LD, r0, lane);
      gemm_nt<T, D, NK>(ts, sQ, sTK, LD, r0, lane);
      gemm_nt<T, D, NK>(acc, sG, sV, LD, r0, lane);  // E
      {
        float w[NK][4];
#pragma unroll
        for (int nt = 0; nt < NK; ++nt) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            ts[nt][e] *= a.sm_scale;
            w[nt][e] = p[nt][e] * (acc[nt][e] - eps[e >> 1]);
          }
        }
        gemm_acc_nn<T, D, BN>(dq, w, sTK, LD, lane);  // gtS tK
      }
#pragma unroll
      for (int nt = 0; nt < NK; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float tsv = ts[nt][e];
          acc[nt][e] = acc[nt][e] * (tsv - mu[e >> 1]) - eps[e >> 1] * tsv;
        }
      }
      gemm_nt<T, D, NK>(acc, sG, sTV, LD, r0, lane);  // + F
    }
    if constexpr (HAS_GO) gemm_nt<T, D, NK>(acc, sGO, sV, LD, r0, lane);  // + dP
#pragma unroll
    for (int nt = 0; nt < NK; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[nt][e] = p[nt][e] * (acc[nt][e] - sub[e >> 1]);
    }
    gemm_acc_nn<T, D, BN>(dq, acc, sK, LD, lane);  // gS K
    __syncthreads();
  }
  cp_async_wait<0>();
  __syncthreads();

  acc_to_smem<T, D>(sQ, LD, r0, lane, dq, a.sm_scale);
  __syncthreads();
  smem_tile_to_global<T, BM, D, NT>(reinterpret_cast<T*>(a.dq) + head_off, sQ, LD, m0, L, tid);
}

template <typename T, int D, bool HAS_GO, bool HAS_GT>
static int launch_bwd_one(const jvpfa_bwd_args& a, cudaStream_t stream) {
  using C = BwdCfg<T, D>;
  const int go = HAS_GO ? 1 : 0, gt = HAS_GT ? 1 : 0;
  const size_t smem_kv = C::smem(gt ? 4 : 2, 1 + go + 2 * gt, true);
  const size_t smem_q = C::smem(1 + go + 2 * gt, gt ? 4 : 2, false);
  auto k1 = bwd_dkdv_kernel<T, D, HAS_GO, HAS_GT>;
  auto k2 = bwd_dq_kernel<T, D, HAS_GO, HAS_GT>;
  cudaError_t e = cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_kv);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_q);
  if (e != cudaSuccess) {
    set_last_cuda_error(e, "cudaFuncSetAttribute(bwd_generic)");
    return JVPFA_ERR_CUDA;
  }
  dim3 grid((a.L + C::OWN - 1) / C::OWN, a.B * a.H);
  k1<<<grid, C::NTHREADS, smem_kv, stream>>>(a);
  k2<<<grid, C::NTHREADS, smem_q, stream>>>(a);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_cuda_error(e, "launch bwd_generic");
    return JVPFA_ERR_CUDA;
  }
  return JVPFA_OK;
}

template <typename T, int D>
static int launch_bwd_d(const jvpfa_bwd_args& a, cudaStream_t s) {
  const bool go = a.go != nullptr, gt = a.gto != nullptr;
  if (go && gt) return launch_bwd_one<T, D, true, true>(a, s);
  if (gt) return launch_bwd_one<T, D, false, true>(a, s);
  return launch_bwd_one<T, D, true, false>(a, s);
}

template <typename T>
static int launch_bwd_t(const jvpfa_bwd_args& a, cudaStream_t s) {
  switch (a.D) {
    case 32:
      return launch_bwd_d<T, 32>(a, s);
    case 64:
      return launch_bwd_d<T, 64>(a, s);
    case 128:
      return launch_bwd_d<T, 128>(a, s);
    default:
      return JVPFA_ERR_SHAPE;
  }
}

int launch_bwd_generic(const jvpfa_bwd_args& a, cudaStream_t s) {
  switch (a.dtype) {
    case JVPFA_BF16:
      return launch_bwd_t<__nv_bfloat16>(a, s);
    case JVPFA_FP16:
      return launch_bwd_t<__half>(a, s);
    case JVPFA_FP32:
      return launch_bwd_t<float>(a, s);
    case JVPFA_FP32_TF32:
      return launch_bwd_t<tf32x1>(a, s);
    default:
      return JVPFA_ERR_DTYPE;
  }
}

}  // namespace jvpfa
