// Fused primal (+ tangent) attention forward for bf16 / fp16 on the Blackwell tensor cores:
// TMA tile loads into 128-byte-swizzled shared memory, tcgen05.mma with accumulators in TMEM,
// warp-specialised online softmax.
//
// CTA = one 128-row query tile of one (batch, head); 6 warps:
//   warp 0      TMA producer (one lane) and owner of the TMEM allocation
//   warp 1      MMA issuer (one lane)
//   warps 2..5  softmax / correction / epilogue: thread <-> one query row <-> one TMEM lane
// TMEM columns (fp32 unless noted):  S [BN] | tS [BN] | O [D] | tO' [D]
//   P (16-bit, BN/2 columns) overwrites the head of S, W = P*tS*scale overwrites the head of tS;
//   both feed the second group of MMAs directly from TMEM as the A operand.
// Per key tile:
//   MMA   : S = Q K^T ; tS = tQ K^T + Q tK^T                       -> commit(s_full)
//   softmax: x = S*scale*log2e (+mask); lazy running max (rescale O, tO' only when the max grows
//            by more than 2^8); P = 2^(x-m); l += sum P; mu += sum W  -> arrive(p_full)
//   MMA   : O += P V ; tO' += W V + P tV                            -> commit(kv_empty[stage])
// Epilogue: O = O/l ; tO = tO'/l - (mu/l) O ; lse = m + log2 l  (same quantities as the
// register-tiled kernel in fwd_generic.cu, which follows jvp_attention.py:125-336, 1011-1033).
//
// With D = 64 a CTA needs 256 TMEM columns and ~97 KB of shared memory, so two CTAs share an SM
// and one CTA's softmax overlaps the other's MMAs.
#include "tc5_common.cuh"

namespace jvpfa {

// [0]: the status word.  [2], [3]: device address of its host-visible mirror (pinned, mapped host memory), written by
// a thread that gives up a wait, so that the host can see a failure without synchronising.
__device__ __align__(16) int g_tc5_status[4] = {0, 0, 0, 0};

namespace {
struct StatusSlot {
  int* dev = nullptr;            // device address of g_tc5_status on that device
  volatile int* mirror = nullptr;  // host address of the mirror (null if it could not be set up)
};
StatusSlot* status_slot() {
  static StatusSlot cache[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  StatusSlot& sl = cache[dev];
  if (!sl.dev) {
    int* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_tc5_status) != cudaSuccess) return nullptr;
    int* host = nullptr;
    int* host_dev = nullptr;
    if (cudaHostAlloc(reinterpret_cast<void**>(&host), sizeof(int), cudaHostAllocMapped) == cudaSuccess) {
      *host = 0;
      if (cudaHostGetDevicePointer(reinterpret_cast<void**>(&host_dev), host, 0) == cudaSuccess &&
          cudaMemcpy(p + 2, &host_dev, sizeof(host_dev), cudaMemcpyHostToDevice) == cudaSuccess) {
        sl.mirror = host;
      } else {
        cudaFreeHost(host);
      }
    }
    (void)cudaGetLastError();  // a missing mirror only costs the early warning
    sl.dev = p;
  }
  return &sl;
}
}  // namespace

// Device address of the status word on the current device (other translation units receive it
// as a kernel argument).  Looked up once per device.
int* tc5_status_device_ptr() {
  StatusSlot* sl = status_slot();
  return sl ? sl->dev : nullptr;
}

// The mirror's value: non-zero once a kernel on the current device has given up a wait (no CUDA call, no
// synchronisation; it can lag behind the device by the kernels still in flight).
int tc5_status_peek() {
  StatusSlot* sl = status_slot();
  return (sl && sl->mirror) ? *sl->mirror : 0;
}

namespace tc5 {

template <int D, bool DUAL>
struct FwdCfg {
  static constexpr int BM = 128;
  static constexpr int BN = 64;
  static constexpr int STAGES = 2;
  static constexpr int NTHREADS = 192;
  static constexpr int Q_BYTES = BM * D * 2;
  static constexpr int KV_BYTES = BN * D * 2;
  static constexpr int N_Q = DUAL ? 2 : 1;
  static constexpr int N_KV = DUAL ? 4 : 2;
  static constexpr int TILE_BYTES = N_Q * Q_BYTES + STAGES * N_KV * KV_BYTES;
  static constexpr int SMEM_BYTES = TILE_BYTES + 256 /*barriers*/ + 1024 /*alignment slack*/;
  // TMEM column map
  static constexpr int COL_S = 0;
  static constexpr int COL_TS = BN;
  static constexpr int COL_O = DUAL ? 2 * BN : BN;
  static constexpr int COL_TO = COL_O + D;
  static constexpr int COLS_USED = DUAL ? 2 * BN + 2 * D : BN + D;
  static constexpr int COLS_ALLOC = COLS_USED <= 128 ? 128 : (COLS_USED <= 256 ? 256 : 512);
  static constexpr int MIN_CTAS = (D <= 64) ? 2 : 1;
};

struct FwdMaps {
  CUtensorMap q, tq, k, tk, v, tv;
};

// MK: 0 = none / causal / key padding; 1 = uint8 mask; 2 = bias of the element type T (the softmax thread
// of a query row reads its 64 mask elements of the tile with 16-byte loads before it waits for the scores;
// key stride 1, 16-byte aligned rows and L % 16 == 0 are the host's responsibility).
template <typename T, int D, bool DUAL, int MK>
__global__ void __launch_bounds__(192, FwdCfg<D, DUAL>::MIN_CTAS)
fwd_tc5_kernel(const jvpfa_fwd_args a, const __grid_constant__ FwdMaps maps) {
  using C = FwdCfg<D, DUAL>;
  constexpr int BM = C::BM, BN = C::BN, STAGES = C::STAGES;
  constexpr int KSTEPS_D = D / 16;   // contraction steps over the head dimension
  constexpr int KSTEPS_N = BN / 16;  // contraction steps over the keys of a tile
  constexpr int HALVES = D / 64;     // 64-column TMA boxes per row

  const bool dead_on_entry = *(volatile int*)&g_tc5_status[0] != 0;  // an earlier bounded wait gave up

  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  unsigned char* smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  unsigned char* sQ = smem;
  unsigned char* sTQ = sQ + C::Q_BYTES;  // DUAL only
  unsigned char* sKV = smem + C::N_Q * C::Q_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::TILE_BYTES);
  uint64_t* q_full = bars + 0;
  uint64_t* kv_full = bars + 1;              // [STAGES]
  uint64_t* kv_empty = bars + 1 + STAGES;    // [STAGES]
  uint64_t* s_full = bars + 1 + 2 * STAGES;
  uint64_t* p_full = s_full + 1;
  uint64_t* o_full = s_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_full + 3);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int L = a.L;
  const int bh = blockIdx.y;
  const int tma_b = bh / a.H, tma_h = bh - tma_b * a.H;  // coordinates in the (D, L, H, B) tensor maps
  const int b = bh / a.H;
  const int mt = (int)gridDim.x - 1 - (int)blockIdx.x;  // heaviest causal tiles first
  const int m0 = mt * BM;
  const bool causal = a.mask.kind == JVPFA_MASK_CAUSAL;
  int n_valid = L;  // keys j < n_valid can attend (before the causal rule)
  if (a.mask.kind == JVPFA_MASK_KVLEN) {
    const int n = a.mask.kv_len[b];
    n_valid = n < 0 ? 0 : (n > L ? L : n);
  }
  int n_end = n_valid;
  if (causal) n_end = min(n_end, m0 + BM);
  const int n_tiles = (n_end + BN - 1) / BN;

  // lse = NaN for this CTA's rows: the results of this launch are not to be trusted
  auto poison = [&]() {
    if (tid < BM && m0 + tid < L) a.lse[(size_t)bh * L + m0 + tid] = poison_f32();
  };
  if (dead_on_entry) {
    poison();
    return;
  }

  if (tid == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(kv_full + s, 1);
      mbar_init(kv_empty + s, 1);
    }
    mbar_init(s_full, 1);
    mbar_init(p_full, 128);
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
  const AbortState ab{abort_flag, &g_tc5_status[0]};

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && n_tiles > 0) {
      prefetch_tmap(&maps.q);
      prefetch_tmap(&maps.k);
      prefetch_tmap(&maps.v);
      mbar_expect_tx(q_full, C::N_Q * C::Q_BYTES);
      for (int hf = 0; hf < HALVES; ++hf) {
        tma_load_4d(sQ + hf * (BM * 128), &maps.q, q_full, hf * 64, m0, tma_h, tma_b);
        if constexpr (DUAL) tma_load_4d(sTQ + hf * (BM * 128), &maps.tq, q_full, hf * 64, m0, tma_h, tma_b);
      }
      for (int it = 0; it < n_tiles; ++it) {
        const int st = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!mbar_wait(kv_empty + st, ph ^ 1, ab, kAbortKvEmpty)) break;
        unsigned char* base = sKV + st * (C::N_KV * C::KV_BYTES);
        mbar_expect_tx(kv_full + st, C::N_KV * C::KV_BYTES);
        const int n0 = it * BN;
        for (int hf = 0; hf < HALVES; ++hf) {
          tma_load_4d(base + hf * (BN * 128), &maps.k, kv_full + st, hf * 64, n0, tma_h, tma_b);
          tma_load_4d(base + C::KV_BYTES + hf * (BN * 128), &maps.v, kv_full + st, hf * 64, n0, tma_h, tma_b);
          if constexpr (DUAL) {
            tma_load_4d(base + 2 * C::KV_BYTES + hf * (BN * 128), &maps.tk, kv_full + st, hf * 64, n0, tma_h, tma_b);
            tma_load_4d(base + 3 * C::KV_BYTES + hf * (BN * 128), &maps.tv, kv_full + st, hf * 64, n0, tma_h, tma_b);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idesc_qk = make_idesc(Fmt<T>::kIdesc, BM, BN, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc(Fmt<T>::kIdesc, BM, D, 0, 1);
      const uint32_t aQ = smem_u32(sQ), aTQ = smem_u32(sTQ);
      // K-major operand, contraction step ks over D
      auto kdesc = [](uint32_t base, int rows, int ks) {
        return make_smem_desc(base + (ks >> 2) * (rows * 128) + (ks & 3) * 32, 16, 1024);
      };
      // MN-major V / tV, contraction step kk over the keys
      auto vdesc = [](uint32_t base, int kk) { return make_smem_desc(base + kk * 2048, BN * 128, 1024); };
      bool ok = mbar_wait(q_full, 0, ab, kAbortQFull);
      for (int it = 0; ok && it < n_tiles; ++it) {
        const int st = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!mbar_wait(kv_full + st, ph, ab, kAbortKvFull)) break;
        tc_fence_after();
        const uint32_t aK = smem_u32(sKV + st * (C::N_KV * C::KV_BYTES));
        const uint32_t aV = aK + C::KV_BYTES, aTK = aK + 2 * C::KV_BYTES, aTV = aK + 3 * C::KV_BYTES;
#pragma unroll
        for (int ks = 0; ks < KSTEPS_D; ++ks)
          umma_ss(tmem + C::COL_S, kdesc(aQ, BM, ks), kdesc(aK, BN, ks), idesc_qk, ks > 0);
        if constexpr (DUAL) {
#pragma unroll
          for (int ks = 0; ks < KSTEPS_D; ++ks)
            umma_ss(tmem + C::COL_TS, kdesc(aTQ, BM, ks), kdesc(aK, BN, ks), idesc_qk, ks > 0);
#pragma unroll
          for (int ks = 0; ks < KSTEPS_D; ++ks)
            umma_ss(tmem + C::COL_TS, kdesc(aQ, BM, ks), kdesc(aTK, BN, ks), idesc_qk, 1);
        }
        tc_commit(s_full);
        if (!mbar_wait(p_full, it & 1, ab, kAbortPFull)) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < KSTEPS_N; ++kk)
          umma_ts(tmem + C::COL_O, tmem + C::COL_S + kk * 8, vdesc(aV, kk), idesc_pv, (it > 0 || kk > 0));
        if constexpr (DUAL) {
#pragma unroll
          for (int kk = 0; kk < KSTEPS_N; ++kk)
            umma_ts(tmem + C::COL_TO, tmem + C::COL_TS + kk * 8, vdesc(aV, kk), idesc_pv, (it > 0 || kk > 0));
#pragma unroll
          for (int kk = 0; kk < KSTEPS_N; ++kk)
            umma_ts(tmem + C::COL_TO, tmem + C::COL_S + kk * 8, vdesc(aTV, kk), idesc_pv, 1);
        }
        tc_commit(kv_empty + st);
      }
      tc_commit(o_full);
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue
    const int quarter = warp & 3;              // TMEM lane quarter this warp may access
    const int row = quarter * 32 + lane;       // tile row == TMEM lane
    const int i = m0 + row;                    // query index
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t tS = tmem + lane_off + C::COL_S, tTS = tmem + lane_off + C::COL_TS;
    const uint32_t tO = tmem + lane_off + C::COL_O, tTO = tmem + lane_off + C::COL_TO;
    const float scale_log2 = a.sm_scale * kLog2e;
    float m_used = -INFINITY, l_run = 0.f, mu_run = 0.f;
    bool alive = true;

    constexpr int MESZ = MK == 1 ? 1 : 2;          // bytes per mask element
    constexpr int MW = MK == 0 ? 1 : 16 * MESZ;    // 32-bit words per row of a 64-key tile
    const unsigned char* mrow = nullptr;
    if constexpr (MK != 0)
      mrow = reinterpret_cast<const unsigned char*>(a.mask.ptr) +
             ((long long)tma_b * a.mask.stride[0] + (long long)tma_h * a.mask.stride[1] +
              (long long)min(i, L - 1) * a.mask.stride[2]) * MESZ;

    for (int it = 0; it < n_tiles; ++it) {
      const int n0 = it * BN;
      uint32_t mw[MW];
      if constexpr (MK != 0) {
#pragma unroll
        for (int j = 0; j < MW / 4; ++j) {
          uint4 r = make_uint4(0u, 0u, 0u, 0u);
          if (n0 + (j + 1) * (16 / MESZ) <= L) r = ldg_nc_v4(mrow + (size_t)n0 * MESZ + 16 * j);
          mw[4 * j] = r.x, mw[4 * j + 1] = r.y, mw[4 * j + 2] = r.z, mw[4 * j + 3] = r.w;
        }
      }
      if (!mbar_wait(s_full, it & 1, ab, kAbortSFull)) {
        alive = false;
        break;
      }
      tc_fence_after();
      uint32_t x0[32], x1[32];
      tmem_ld32(tS, x0);
      tmem_ld32(tS + 32, x1);
      tmem_wait_ld();
      const bool partial = (causal && n0 + BN - 1 > m0) || (n0 + BN > n_valid);
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        float v0 = __uint_as_float(x0[c]) * scale_log2;
        float v1 = __uint_as_float(x1[c]) * scale_log2;
        if constexpr (MK == 1) {  // byte c and byte 32 + c of the row's 64
          if (!((mw[c >> 2] >> ((c & 3) * 8)) & 0xffu)) v0 = -INFINITY;
          if (!((mw[8 + (c >> 2)] >> ((c & 3) * 8)) & 0xffu)) v1 = -INFINITY;
        }
        if constexpr (MK == 2) {  // scores are in log2 units: bias * log2(e)
          v0 = fmaf(unpack1<T>((mw[c >> 1] >> ((c & 1) * 16)) & 0xffffu), kLog2e, v0);
          v1 = fmaf(unpack1<T>((mw[16 + (c >> 1)] >> ((c & 1) * 16)) & 0xffffu), kLog2e, v1);
        }
        if (partial) {
          const int j0 = n0 + c, j1 = n0 + 32 + c;
          if (j0 >= n_valid || (causal && j0 > i)) v0 = -INFINITY;
          if (j1 >= n_valid || (causal && j1 > i)) v1 = -INFINITY;
        }
        x0[c] = __float_as_uint(v0);
        x1[c] = __float_as_uint(v1);
        mx = fmaxf(mx, fmaxf(v0, v1));
      }
      // Lazy running max: keep the old reference while the new maximum is at most 2^8 above it.
      const bool grow = mx > m_used + 8.f;
      float alpha = 1.f;
      if (grow) {
        alpha = fast_exp2(m_used - mx);
        m_used = mx;
      }
      const float m_eff = (m_used == -INFINITY) ? 0.f : m_used;
      if (it > 0 && __any_sync(0xffffffffu, grow)) {
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(tO + 32 * c, r);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * alpha);
          tmem_st32(tO + 32 * c, r);
          if constexpr (DUAL) {
            tmem_ld32(tTO + 32 * c, r);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * alpha);
            tmem_st32(tTO + 32 * c, r);
          }
        }
      }
      float ls = 0.f;
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        const float p0 = fast_exp2(__uint_as_float(x0[c]) - m_eff);
        const float p1 = fast_exp2(__uint_as_float(x1[c]) - m_eff);
        x0[c] = __float_as_uint(p0);
        x1[c] = __float_as_uint(p1);
        ls += p0 + p1;
      }
      l_run = l_run * alpha + ls;
      if constexpr (DUAL) {
        float ms = 0.f;
        uint32_t t[32];
        uint32_t wp[16];
        tmem_ld32(tTS, t);
        tmem_wait_ld();
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          const float w0 = __uint_as_float(x0[2 * c]) * (__uint_as_float(t[2 * c]) * a.sm_scale);
          const float w1 = __uint_as_float(x0[2 * c + 1]) * (__uint_as_float(t[2 * c + 1]) * a.sm_scale);
          ms += w0 + w1;
          wp[c] = Elem<T>::pack(w0, w1);
        }
        tmem_ld32(tTS + 32, t);  // second half is read before the first packed half is written below
        tmem_wait_ld();
        tmem_st16(tTS, wp);
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          const float w0 = __uint_as_float(x1[2 * c]) * (__uint_as_float(t[2 * c]) * a.sm_scale);
          const float w1 = __uint_as_float(x1[2 * c + 1]) * (__uint_as_float(t[2 * c + 1]) * a.sm_scale);
          ms += w0 + w1;
          wp[c] = Elem<T>::pack(w0, w1);
        }
        tmem_st16(tTS + 16, wp);
        mu_run = mu_run * alpha + ms;
      }
      {
        uint32_t pp[32];
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          pp[c] = Elem<T>::pack(__uint_as_float(x0[2 * c]), __uint_as_float(x0[2 * c + 1]));
          pp[16 + c] = Elem<T>::pack(__uint_as_float(x1[2 * c]), __uint_as_float(x1[2 * c + 1]));
        }
        tmem_st32(tS, pp);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(p_full);
    }

    // ---- epilogue ----
    if (alive && n_tiles > 0) alive = mbar_wait(o_full, 0, ab, kAbortOFull);
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
        if (n_tiles > 0) {
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
          if (n_tiles > 0) {
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

  // ---- teardown: every thread arrives here, with or without an abort ----
  tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0) poison();
  if (warp == 0) {
    if (*abort_flag != 0) {
      // Something gave up: give copies and MMAs that may still be in flight time to land before
      // the TMEM columns go back to the allocator.
      const long long t0 = clock64();
      while (clock64() - t0 < (1ll << 22)) {
      }
    }
    tc_fence_after();
    tmem_dealloc(tmem, C::COLS_ALLOC);
  }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

bool encode_map4d(CUtensorMap* m, CUtensorMapDataType dt, const void* ptr, int D, int L, int H, int B, const int64_t* st,
                  int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  const bool dense = st == nullptr || (st[0] == 0 && st[1] == 0 && st[2] == 0);
  const cuuint64_t sb = dense ? (cuuint64_t)H * L * D : (cuuint64_t)st[0];
  const cuuint64_t sh = dense ? (cuuint64_t)L * D : (cuuint64_t)st[1];
  const cuuint64_t sl = dense ? (cuuint64_t)D : (cuuint64_t)st[2];
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)L, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {sl * 2, sh * 2, sb * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(m, dt, 4, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// Row-major fp32 (B, H, L, D) tensor as a 4-D map with 32-column (128-byte) swizzled boxes: target of TMA reductions.
bool encode_map4d_f32(CUtensorMap* m, const void* ptr, int D, int L, int H, int B, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)L, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)D * 4, (cuuint64_t)L * D * 4, (cuuint64_t)H * L * D * 4};
  cuuint32_t box[4] = {32, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

bool encode_map4(CUtensorMap* m, CUtensorMapDataType dt, const void* ptr, int L, int H, int B, const int64_t* st,
                 int box_rows) {
  return encode_map4d(m, dt, ptr, 64, L, H, B, st, box_rows);
}

template <typename T, int D, bool DUAL, int MK>
static int launch_one(const jvpfa_fwd_args& a, cudaStream_t stream) {
  using C = FwdCfg<D, DUAL>;
  FwdMaps maps;
  const long long BH = (long long)a.B * a.H;
  const CUtensorMapDataType dt = Fmt<T>::kTma;
  bool ok = encode_map4d(&maps.q, dt, a.q, D, a.L, a.H, a.B, a.in_stride, C::BM) && encode_map4d(&maps.k, dt, a.k, D, a.L, a.H, a.B, a.in_stride, C::BN) &&
            encode_map4d(&maps.v, dt, a.v, D, a.L, a.H, a.B, a.in_stride, C::BN);
  if (DUAL)
    ok = ok && encode_map4d(&maps.tq, dt, a.tq, D, a.L, a.H, a.B, a.in_stride, C::BM) && encode_map4d(&maps.tk, dt, a.tk, D, a.L, a.H, a.B, a.in_stride, C::BN) &&
         encode_map4d(&maps.tv, dt, a.tv, D, a.L, a.H, a.B, a.in_stride, C::BN);
  else
    maps.tq = maps.tk = maps.tv = maps.q;
  if (!ok) {
    set_last_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled");
    return JVPFA_ERR_CUDA;
  }
  auto kern = fwd_tc5_kernel<T, D, DUAL, MK>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
  if (e != cudaSuccess) {
    set_last_cuda_error(e, "cudaFuncSetAttribute(fwd_tc5)");
    return JVPFA_ERR_CUDA;
  }
  dim3 grid((a.L + C::BM - 1) / C::BM, a.B * a.H);
  kern<<<grid, C::NTHREADS, C::SMEM_BYTES, stream>>>(a, maps);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_cuda_error(e, "launch fwd_tc5");
    return JVPFA_ERR_CUDA;
  }
  return JVPFA_OK;
}

template <typename T>
static int launch_t(const jvpfa_fwd_args& a, cudaStream_t s) {
  const bool dual = a.tq != nullptr;
  if (a.D == 64) return dual ? launch_one<T, 64, true, 0>(a, s) : launch_one<T, 64, false, 0>(a, s);
  return JVPFA_ERR_UNSUPPORTED;  // head dimension 128 has its own kernel
}

}  // namespace tc5

bool fwd_tc5_eligible(const jvpfa_fwd_args& a) {
  if (a.dtype != JVPFA_BF16 && a.dtype != JVPFA_FP16) return false;
  if (a.D != 64 && a.D != 128) return false;
  const int k = a.mask.kind;
  if (k == JVPFA_MASK_NONE || k == JVPFA_MASK_CAUSAL || k == JVPFA_MASK_KVLEN) return true;
  // Boolean masks and bias: the softmax threads read 16-byte pieces of mask rows
  if ((a.D == 64 && !(a.sm_scale > 0.f)) || (a.L & 15) != 0) return false;
  if (k == JVPFA_MASK_BIAS && a.mask.bias_dtype != a.dtype) return false;
  const long long esz = k == JVPFA_MASK_BOOL ? 1 : 2;
  if (a.mask.stride[3] != 1 || (reinterpret_cast<uintptr_t>(a.mask.ptr) & 15u) != 0) return false;
  for (int d = 0; d < 3; ++d)
    if (a.mask.stride[d] < 0 || ((a.mask.stride[d] * esz) & 15) != 0) return false;
  return true;
}

int launch_fwd_tc5(const jvpfa_fwd_args& a, cudaStream_t s) {
  // Query-tile-pair kernel (fwd_tc5_pair64.cu); it takes the row maximum before scaling and therefore
  // needs a positive softmax scale.
  if (a.D == 64 && a.sm_scale > 0.f) return launch_fwd_tc5_pair64(a, s);
  // Head dimension 128: score products of the next key tile under the softmax of this one (fwd_tc5_pipe128.cu).
  if (a.D == 128) return launch_fwd_tc5_pipe128(a, s);
  return a.dtype == JVPFA_BF16 ? tc5::launch_t<__nv_bfloat16>(a, s) : tc5::launch_t<__half>(a, s);
}

int tc5_read_status(int* out, int clear) {
  StatusSlot* sl = status_slot();
  if (!sl) {
    set_last_cuda_error(cudaErrorUnknown, "status word address");
    return JVPFA_ERR_CUDA;
  }
  int v = 0;
  cudaError_t e = cudaMemcpy(&v, sl->dev, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) {
    set_last_cuda_error(e, "cudaMemcpy(status)");
    return JVPFA_ERR_CUDA;
  }
  if (clear && v != 0) {
    const int zero = 0;
    e = cudaMemcpy(sl->dev, &zero, sizeof(int), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
      set_last_cuda_error(e, "cudaMemcpy(status)");
      return JVPFA_ERR_CUDA;
    }
    if (sl->mirror) *sl->mirror = 0;
  }
  *out = v;
  return JVPFA_OK;
}

// Puts `code` into the status word and its mirror from the host, as a kernel that gave up a wait would.
int tc5_inject_status(int code) {
  StatusSlot* sl = status_slot();
  if (!sl) {
    set_last_cuda_error(cudaErrorUnknown, "status word address");
    return JVPFA_ERR_CUDA;
  }
  cudaError_t e = cudaMemcpy(sl->dev, &code, sizeof(int), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    set_last_cuda_error(e, "cudaMemcpy(status)");
    return JVPFA_ERR_CUDA;
  }
  if (sl->mirror) *sl->mirror = code;
  return JVPFA_OK;
}

}  // namespace jvpfa
