// Fused primal (+ tangent) attention forward on warp-level tensor-core MMAs.
//
// One CTA of 4 warps owns a 64-row query tile of one (batch, head); each warp owns 16 rows.
// K, tK, V, tV tiles stream through a two-stage cp.async ring in shared memory.  Per tile the
// warp forms S = Q K^T and tS = tQ K^T + Q tK^T in registers, applies the mask / bias, runs the
// online softmax (running max m, denominator l and mu = sum P*tS) and feeds P and P*tS straight
// from the accumulator registers into the second set of MMAs (O += P V, tO' += (P*tS) V + P tV).
// Epilogue: O = acc/l, tO = tO'/l - (mu/l) O, lse = m + log2(l)  (base 2, scaled scores).
//
// Math follows upstream's _attn_fwd_inner (jvp_flash_attention/jvp_attention.py:125-336) and the
// epilogue at jvp_attention.py:1011-1033, with two deliberate differences: the additive bias
// is applied as scale*QK^T + bias (SDPA semantics; upstream scales the bias too,
// jvp_attention.py:247-251), and boolean masking uses -inf rather than adding -100.
#include "common.cuh"

namespace jvpfa {

template <typename T, int D>
struct FwdCfg {
  static constexpr int BM = 64;
  static constexpr int BN = (!Elem<T>::k16 || D > 64) ? 32 : 64;
  static constexpr int LD = D + Elem<T>::kPad;
  static constexpr int NTHREADS = 128;
  static constexpr int STAGES = 2;
  static constexpr size_t smem(bool dual) {
    return sizeof(T) * ((size_t)BM * LD * (dual ? 2 : 1) + (size_t)STAGES * BN * LD * (dual ? 4 : 2));
  }
};

template <typename T, int D, bool DUAL>
__global__ void __launch_bounds__(128) fwd_generic_kernel(const jvpfa_fwd_args a) {
  using C = FwdCfg<T, D>;
  constexpr int BM = C::BM, BN = C::BN, LD = C::LD, NT = C::NTHREADS;
  constexpr int KS = Elem<T>::kKStep;
  constexpr int NS = BN / 8;   // score n-tiles per warp row-strip
  constexpr int ND = D / 8;    // output n-tiles
  constexpr int NKV = DUAL ? 4 : 2;

  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* sQ = reinterpret_cast<T*>(smem_raw);
  T* sTQ = sQ + BM * LD;  // only valid when DUAL
  T* sKV = sQ + BM * LD * (DUAL ? 2 : 1);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int L = a.L;
  const int bh = blockIdx.y;
  const int b = bh / a.H, h = bh - b * a.H;
  // Heaviest causal tiles (largest m0) are scheduled first.
  const int mt = (int)gridDim.x - 1 - (int)blockIdx.x;
  const int m0 = mt * BM;

  const size_t head_off = (size_t)bh * L * D;
  // the six inputs may share a strided (batch, head, row) layout (in_stride, elements; all zero = row-major)
  const bool strided = (a.in_stride[0] | a.in_stride[1] | a.in_stride[2]) != 0;
  const long long in_off = strided ? (long long)b * a.in_stride[0] + (long long)h * a.in_stride[1] : (long long)head_off;
  const long long in_rs = strided ? a.in_stride[2] : D;
  const T* gQ = reinterpret_cast<const T*>(a.q) + in_off;
  const T* gK = reinterpret_cast<const T*>(a.k) + in_off;
  const T* gV = reinterpret_cast<const T*>(a.v) + in_off;
  const T* gTQ = DUAL ? reinterpret_cast<const T*>(a.tq) + in_off : nullptr;
  const T* gTK = DUAL ? reinterpret_cast<const T*>(a.tk) + in_off : nullptr;
  const T* gTV = DUAL ? reinterpret_cast<const T*>(a.tv) + in_off : nullptr;

  const MaskView mv = make_mask_view(a.mask, b, h, L);

  int n_end = L;
  if (mv.kind == JVPFA_MASK_CAUSAL) n_end = min(L, m0 + BM);
  if (mv.kind == JVPFA_MASK_KVLEN) n_end = min(L, mv.kv_len);
  const int n_tiles = (n_end + BN - 1) / BN;

  auto stage_kv = [&](int stage, int n0) {
    T* base = sKV + (size_t)stage * NKV * BN * LD;
    stage_tile<T, BN, D, NT>(base, gK, n0, L, tid, in_rs);
    stage_tile<T, BN, D, NT>(base + BN * LD, gV, n0, L, tid, in_rs);
    if constexpr (DUAL) {
      stage_tile<T, BN, D, NT>(base + 2 * BN * LD, gTK, n0, L, tid, in_rs);
      stage_tile<T, BN, D, NT>(base + 3 * BN * LD, gTV, n0, L, tid, in_rs);
    }
  };

  // Prologue: Q (+tQ) and the first K/V tile in one cp.async group.
  stage_tile<T, BM, D, NT>(sQ, gQ, m0, L, tid, in_rs);
  if constexpr (DUAL) stage_tile<T, BM, D, NT>(sTQ, gTQ, m0, L, tid, in_rs);
  if (n_tiles > 0) stage_kv(0, 0);
  cp_async_commit();

  const float scale_log2 = a.sm_scale * kLog2e;
  const int r0 = warp * 16;
  const int row_lo = m0 + r0 + g, row_hi = row_lo + 8;

  float acc_o[ND][4];
  float acc_t[DUAL ? ND : 1][4];
#pragma unroll
  for (int i = 0; i < ND; ++i) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      acc_o[i][j] = 0.f;
      if constexpr (DUAL) acc_t[i][j] = 0.f;
    }
  }
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};
  float mu_run[2] = {0.f, 0.f};

  for (int it = 0; it < n_tiles; ++it) {
    const int n0 = it * BN;
    if (it + 1 < n_tiles) stage_kv((it + 1) & 1, n0 + BN);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();

    const T* sK = sKV + (size_t)(it & 1) * NKV * BN * LD;
    const T* sV = sK + BN * LD;
    const T* sTK = sK + 2 * BN * LD;
    const T* sTV = sK + 3 * BN * LD;

    // ---- scores ----
    float s[NS][4];
    float ts[DUAL ? NS : 1][4];
#pragma unroll
    for (int i = 0; i < NS; ++i) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        s[i][j] = 0.f;
        if constexpr (DUAL) ts[i][j] = 0.f;
      }
    }
#pragma unroll
    for (int k0 = 0; k0 < D; k0 += KS) {
      FragA<T> fq, ftq;
      load_a<T>(fq, sQ, LD, r0, k0, lane);
      if constexpr (DUAL) load_a<T>(ftq, sTQ, LD, r0, k0, lane);
#pragma unroll
      for (int nt = 0; nt < NS; ++nt) {
        FragB<T> fk;
        load_b_nt<T>(fk, sK, LD, nt * 8, k0, lane);
        mma<T>(s[nt], fq, fk);
        if constexpr (DUAL) {
          FragB<T> ftk;
          load_b_nt<T>(ftk, sTK, LD, nt * 8, k0, lane);
          mma<T>(ts[nt], ftq, fk);
          mma<T>(ts[nt], fq, ftk);
        }
      }
    }

    // ---- mask / bias, move to the base-2 domain ----
    const bool full_tile = (mv.kind == JVPFA_MASK_NONE && n0 + BN <= L && m0 + BM <= L) ||
                           (mv.kind == JVPFA_MASK_CAUSAL && n0 + BN - 1 <= m0 && m0 + BM <= L) ||
                           (mv.kind == JVPFA_MASK_KVLEN && n0 + BN <= mv.kv_len && m0 + BM <= L);
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < NS; ++nt) {
#pragma unroll
      for (int r = 0; r < 2; ++r) {  // accumulator elements 2r, 2r+1: row_lo / row_hi, keys j, j + 1
        const int i = r == 0 ? row_lo : row_hi;
        const int j = n0 + nt * 8 + 2 * t;
        bool ok[2] = {true, true};
        float bias[2] = {0.f, 0.f};
        if (!full_tile) mv.pair(i, j, ok, bias);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int e = 2 * r + c;
          float x = s[nt][e] * scale_log2;
          if (!full_tile) {
            if (ok[c]) {
              x += bias[c] * kLog2e;
            } else {
              x = -INFINITY;
              if constexpr (DUAL) ts[nt][e] = 0.f;
            }
          }
          s[nt][e] = x;
          mx[r] = fmaxf(mx[r], x);
        }
      }
    }
    float alpha[2], m_use[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = quad_max(mx[r]);
      const float m_new = fmaxf(m_run[r], mx[r]);
      m_use[r] = (m_new == -INFINITY) ? 0.f : m_new;
      alpha[r] = exp2f(m_run[r] - m_use[r]);  // m_run = -inf -> 0
      m_run[r] = m_new;
    }
    float ls[2] = {0.f, 0.f}, ms[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < NS; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float p = exp2f(s[nt][e] - m_use[e >> 1]);
        s[nt][e] = p;
        ls[e >> 1] += p;
        if constexpr (DUAL) {
          const float w = p * (ts[nt][e] * a.sm_scale);
          ts[nt][e] = w;
          ms[e >> 1] += w;
        }
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      l_run[r] = l_run[r] * alpha[r] + quad_sum(ls[r]);
      if constexpr (DUAL) mu_run[r] = mu_run[r] * alpha[r] + quad_sum(ms[r]);
    }
#pragma unroll
    for (int dt = 0; dt < ND; ++dt) {
      acc_o[dt][0] *= alpha[0];
      acc_o[dt][1] *= alpha[0];
      acc_o[dt][2] *= alpha[1];
      acc_o[dt][3] *= alpha[1];
      if constexpr (DUAL) {
        acc_t[dt][0] *= alpha[0];
        acc_t[dt][1] *= alpha[0];
        acc_t[dt][2] *= alpha[1];
        acc_t[dt][3] *= alpha[1];
      }
    }

    // ---- second MMAs: contraction over the keys of this tile ----
    if constexpr (Elem<T>::k16) {
#pragma unroll
      for (int kk = 0; kk < BN / KS; ++kk) {
        FragA<T> fp, fw;
        a_from_acc<T>(fp, s, kk);
        if constexpr (DUAL) a_from_acc<T>(fw, ts, kk);
#pragma unroll
        for (int dt = 0; dt < ND; ++dt) {
          FragB<T> fv;
          load_b_nn<T>(fv, sV, LD, kk * KS, dt * 8, lane);
          mma<T>(acc_o[dt], fp, fv);
          if constexpr (DUAL) {
            FragB<T> ftv;
            load_b_nn<T>(ftv, sTV, LD, kk * KS, dt * 8, lane);
            mma<T>(acc_t[dt], fw, fv);
            mma<T>(acc_t[dt], fp, ftv);
          }
        }
      }
    } else {
      // fp32: the tensor core adds into its fp32 accumulator with truncation; over a thousand keys
      // that bias reaches ~1e-5.  This tile's contribution is therefore accumulated in a fresh
      // register tile (32 output columns at a time) and added to the running sums once, rounded.
#pragma unroll
      for (int d0 = 0; d0 < ND; d0 += 4) {
        float to_[4][4], tt_[DUAL ? 4 : 1][4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          to_[i][0] = to_[i][1] = to_[i][2] = to_[i][3] = 0.f;
          if constexpr (DUAL) tt_[i][0] = tt_[i][1] = tt_[i][2] = tt_[i][3] = 0.f;
        }
#pragma unroll
        for (int kk = 0; kk < BN / KS; ++kk) {
          FragA<T> fp, fw;
          a_from_acc<T>(fp, s, kk);
          if constexpr (DUAL) a_from_acc<T>(fw, ts, kk);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            FragB<T> fv;
            load_b_nn<T>(fv, sV, LD, kk * KS, (d0 + i) * 8, lane);
            mma<T>(to_[i], fp, fv);
            if constexpr (DUAL) {
              FragB<T> ftv;
              load_b_nn<T>(ftv, sTV, LD, kk * KS, (d0 + i) * 8, lane);
              mma<T>(tt_[i], fw, fv);
              mma<T>(tt_[i], fp, ftv);
            }
          }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            acc_o[d0 + i][e] += to_[i][e];
            if constexpr (DUAL) acc_t[d0 + i][e] += tt_[i][e];
          }
        }
      }
    }
    __syncthreads();  // every warp is done with this stage before it is refilled
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- epilogue ----
  float inv_l[2], mu_n[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const bool empty = !(l_run[r] > 0.f);
    inv_l[r] = empty ? 0.f : 1.f / l_run[r];
    mu_n[r] = DUAL ? mu_run[r] * inv_l[r] : 0.f;
    const int row = r == 0 ? row_lo : row_hi;
    if (t == 0 && row < L) {
      a.lse[(size_t)bh * L + row] = empty ? INFINITY : (m_run[r] + log2f(l_run[r]));
      if constexpr (DUAL) a.mu[(size_t)bh * L + row] = mu_n[r];
    }
  }
  // Stage the output tiles through the (now idle) Q / tQ buffers for 16-byte coalesced stores.
#pragma unroll
  for (int dt = 0; dt < ND; ++dt) {
    float o0 = acc_o[dt][0] * inv_l[0], o1 = acc_o[dt][1] * inv_l[0];
    float o2 = acc_o[dt][2] * inv_l[1], o3 = acc_o[dt][3] * inv_l[1];
    const int c = dt * 8 + 2 * t;
    T* plo = sQ + (r0 + g) * LD + c;
    T* phi = plo + 8 * LD;
    plo[0] = Elem<T>::from_float(o0);
    plo[1] = Elem<T>::from_float(o1);
    phi[0] = Elem<T>::from_float(o2);
    phi[1] = Elem<T>::from_float(o3);
    if constexpr (DUAL) {
      T* qlo = sTQ + (r0 + g) * LD + c;
      T* qhi = qlo + 8 * LD;
      qlo[0] = Elem<T>::from_float(acc_t[dt][0] * inv_l[0] - mu_n[0] * o0);
      qlo[1] = Elem<T>::from_float(acc_t[dt][1] * inv_l[0] - mu_n[0] * o1);
      qhi[0] = Elem<T>::from_float(acc_t[dt][2] * inv_l[1] - mu_n[1] * o2);
      qhi[1] = Elem<T>::from_float(acc_t[dt][3] * inv_l[1] - mu_n[1] * o3);
    }
  }
  __syncthreads();
  {
    constexpr int VEC = 16 / (int)sizeof(T);
    constexpr int VPR = D / VEC;
    T* gO = reinterpret_cast<T*>(a.o) + head_off;
    T* gTO = DUAL ? reinterpret_cast<T*>(a.to) + head_off : nullptr;
    for (int idx = tid; idx < BM * VPR; idx += NT) {
      const int r = idx / VPR, c = (idx - r * VPR) * VEC;
      const int row = m0 + r;
      if (row < L) {
        *reinterpret_cast<uint4*>(gO + (size_t)row * D + c) = *reinterpret_cast<const uint4*>(sQ + r * LD + c);
        if constexpr (DUAL)
          *reinterpret_cast<uint4*>(gTO + (size_t)row * D + c) =
              *reinterpret_cast<const uint4*>(sTQ + r * LD + c);
      }
    }
  }
}

template <typename T, int D, bool DUAL>
static int launch_one(const jvpfa_fwd_args& a, cudaStream_t stream) {
  using C = FwdCfg<T, D>;
  const size_t smem = C::smem(DUAL);
  auto kern = fwd_generic_kernel<T, D, DUAL>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    set_last_cuda_error(e, "cudaFuncSetAttribute(fwd_generic)");
    return JVPFA_ERR_CUDA;
  }
  dim3 grid((a.L + C::BM - 1) / C::BM, a.B * a.H);
  kern<<<grid, C::NTHREADS, smem, stream>>>(a);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_cuda_error(e, "launch fwd_generic");
    return JVPFA_ERR_CUDA;
  }
  return JVPFA_OK;
}

template <typename T, int D>
static int launch_d(const jvpfa_fwd_args& a, cudaStream_t s) {
  return a.tq ? launch_one<T, D, true>(a, s) : launch_one<T, D, false>(a, s);
}

template <typename T>
static int launch_t(const jvpfa_fwd_args& a, cudaStream_t s) {
  switch (a.D) {
    case 32:
      return launch_d<T, 32>(a, s);
    case 64:
      return launch_d<T, 64>(a, s);
    case 128:
      return launch_d<T, 128>(a, s);
    default:
      return JVPFA_ERR_SHAPE;
  }
}

int launch_fwd_generic(const jvpfa_fwd_args& a, cudaStream_t s) {
  switch (a.dtype) {
    case JVPFA_BF16:
      return launch_t<__nv_bfloat16>(a, s);
    case JVPFA_FP16:
      return launch_t<__half>(a, s);
    case JVPFA_FP32:
      return launch_t<float>(a, s);
    case JVPFA_FP32_TF32:
      return launch_t<tf32x1>(a, s);
    default:
      return JVPFA_ERR_DTYPE;
  }
}

}  // namespace jvpfa
