// Fused primal (+ tangent) attention forward for head dimension 64 (bf16 / fp16; none, causal,
// key padding, and -- template parameter MK -- boolean masks and additive bias) on tcgen05 / TMA / TMEM: the variant of fwd_tc5.cu tuned to how the B200 tensor
// pipe is fed.  A single thread can issue a tcgen05.mma only about every 58-70 cycles whatever
// N <= 128 is, so the kernel (a) halves the instruction count by letting one N=128 instruction
// cover two accumulators that share the A operand and whose B tiles are neighbours in shared
// memory, and (b) issues from two warps with disjoint accumulator chains:
//
//   issuer A:  [S | tS] = Q [K ; tK]^T  (N=128) ;  tS += tQ K^T  (N=64)         -> s_full
//   issuer B:  [O | tO'] += P [V | tV]  (N=128) ;  tO' += W V    (N=64)         -> kv_empty[stage]
//
// Work item = one 128-row query tile of one (batch, head).  The CTAs are persistent (two per SM):
// each walks a static list of items, so barriers and TMEM are set up once, the next item's Q and
// first key tiles are on their way while the current item finishes.  7 warps: TMA producer, issuer A, issuer B,
// four softmax / epilogue warps (thread <-> query row <-> TMEM lane).  TMEM columns:
//   S [64] | tS [64] | O [64] | tO' [64]   (256 columns -> two CTAs per SM)
// P and W = P*tS*scale are written as packed 16-bit values over the head of S and tS and feed
// issuer B's MMAs as TMEM A operands.  Online softmax with lazy rescaling as in fwd_tc5.cu; the
// per-row arithmetic uses packed fp32x2 instructions.
//
// Masks and bias (MK = 1: uint8 mask, MK = 2: bias of the element type T).  A softmax thread owns one
// query row, so its share of a mask tile is 64 consecutive elements of one mask row: 64 or 128 bytes,
// fetched as 16-byte read-only loads that are issued before the thread waits for the tile's scores,
// and applied while the scores are scaled.  Broadcast dimensions are strides of zero.  The key
// stride must be 1, every row start 16-byte aligned and L a multiple of 16 (checked by the host
// code, which otherwise sends the request to the register-tiled kernels).
//
// Tile skipping (MK = 3: uint8 mask with a tile bitmap): mask_tile_live holds one bit per 128-query x 64-key tile of the
// mask, set when the tile has a true entry (written by jvpfa_mask_tiles).  Every role reads the
// item's words and steps over dead tiles in the same way, so the barrier phases (counted in live
// tiles) stay in step; an item without a live tile takes the "no key" path.  It is an instantiation of
// its own so that the kernels without a bitmap keep their plain tile loops.
#include "tc5_common.cuh"

namespace jvpfa {
namespace tc5 {

template <bool DUAL>
struct Fwd64Cfg {
  static constexpr int D = 64;
  static constexpr int BM = 128;
  static constexpr int BN = 64;
  static constexpr int STAGES = 2;
  static constexpr int NTHREADS = 224;
  static constexpr int Q_BYTES = BM * D * 2;   // 16 KiB
  static constexpr int KV_BYTES = BN * D * 2;  // 8 KiB
  static constexpr int N_Q = DUAL ? 2 : 1;
  static constexpr int N_KV = DUAL ? 4 : 2;
  // stage layout: K, tK, V, tV (DUAL) or K, V
  static constexpr int SLOT_K = 0, SLOT_TK = 1, SLOT_V = DUAL ? 2 : 1, SLOT_TV = 3;
  static constexpr int TILE_BYTES = N_Q * Q_BYTES + STAGES * N_KV * KV_BYTES;
  static constexpr int SMEM_BYTES = TILE_BYTES + 256 + 1024;
  static constexpr int COL_S = 0;
  static constexpr int COL_TS = 64;
  static constexpr int COL_O = DUAL ? 128 : 64;
  static constexpr int COL_TO = 192;
  static constexpr int COLS_ALLOC = DUAL ? 256 : 128;
};

struct Fwd64Maps {
  CUtensorMap q, tq, k, tk, v, tv;
};

__device__ __forceinline__ float2 ff2(uint32_t a, uint32_t b) { return make_float2(__uint_as_float(a), __uint_as_float(b)); }

// One work item of the persistent loop: a 128-row query tile of one (batch, head).
struct FwdItem {
  int bh, b, h, m0, n_valid, n_tiles;
  const unsigned long long* live;  // MK = 3: this item's words of the tile bitmap, or nullptr
};

// Walks an item's key tiles, telling the live ones (bit t of the item's bitmap words) from the dead.
struct LiveTiles {
  const unsigned long long* words;
  unsigned long long bits;
  __device__ __forceinline__ explicit LiveTiles(const unsigned long long* w) : words(w), bits(~0ull) {}
  __device__ __forceinline__ bool operator()(int t) {
    if (words == nullptr) return true;
    if ((t & 63) == 0) bits = __ldg(words + (t >> 6));
    return (bits >> (t & 63)) & 1ull;
  }
};

template <typename T, bool DUAL, int MK>
__global__ void __launch_bounds__(224, 2)
fwd_tc5_d64_kernel(const jvpfa_fwd_args a, const __grid_constant__ Fwd64Maps maps, int* status) {
  using C = Fwd64Cfg<DUAL>;
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
  uint64_t* s_full = bars + 1 + 2 * STAGES;
  uint64_t* p_full = s_full + 1;
  uint64_t* o_full = s_full + 2;
  uint64_t* q_empty = s_full + 3;  // issuer A has read the item's Q tiles
  uint64_t* o_free = s_full + 4;   // the epilogue has read the item's accumulators
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_full + 5);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int L = a.L;
  const int BH = a.B * a.H;
  const bool causal = a.mask.kind == JVPFA_MASK_CAUSAL;
  const int n_q_tiles = (L + BM - 1) / BM;
  const int n_items = n_q_tiles * BH;
  const int G = (int)gridDim.x, cta = (int)blockIdx.x;
  const int k_max = (n_items + G - 1) / G;

  // Item k of this CTA.  The CTAs stay resident (two per SM) and walk a static list: items are ranked
  // heaviest first (for causal masks the last query tile is the longest) and dealt in serpentine order.
  auto get_item = [&](int k, FwdItem& it) -> bool {
    const int w = k * G + ((k & 1) ? (G - 1 - cta) : cta);
    if (w >= n_items) return false;
    if (causal) {  // heaviest query tiles first, over all heads
      const int rank = w / BH;
      it.bh = w - rank * BH;
      it.m0 = (n_q_tiles - 1 - rank) * BM;
    } else {  // equal weights: the query tiles of a head run side by side and share its K / V in L2
      it.bh = w / n_q_tiles;
      it.m0 = (w - it.bh * n_q_tiles) * BM;
    }
    it.b = it.bh / a.H;
    it.h = it.bh - it.b * a.H;
    it.n_valid = L;
    if (a.mask.kind == JVPFA_MASK_KVLEN) {
      const int n = a.mask.kv_len[it.b];
      it.n_valid = n < 0 ? 0 : (n > L ? L : n);
    }
    int n_end = it.n_valid;
    if (causal) n_end = min(n_end, it.m0 + BM);
    it.n_tiles = (n_end + BN - 1) / BN;
    it.live = nullptr;
    if constexpr (MK == 3) {
      {
        // the bitmap has the mask's own extents: broadcast dimensions (stride 0) have one entry
        const int n_words = (it.n_tiles + 63) >> 6;
        const long long hm = (a.mask.stride[0] ? (long long)it.b * (a.mask.stride[1] ? a.H : 1) : 0) +
                             (a.mask.stride[1] ? it.h : 0);
        const long long qm = a.mask.stride[2] ? hm * n_q_tiles + it.m0 / BM : hm;
        it.live = reinterpret_cast<const unsigned long long*>(a.mask_tile_live) + qm * n_words;
        bool any = false;
        for (int w = 0; w < n_words; ++w) any = any || __ldg(it.live + w) != 0ull;
        if (!any) it.n_tiles = 0;  // nothing to attend to: zeros and lse = +inf, as for kv_len = 0
      }
    }
    return true;
  };

  if (tid == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(kv_full + s, 1);
      mbar_init(kv_empty + s, 1);
    }
    mbar_init(s_full, 1);
    mbar_init(p_full, 128);
    mbar_init(o_full, 1);
    mbar_init(q_empty, 1);
    mbar_init(o_free, 128);
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

  // Barrier phases run on across the items: g counts the key tiles of all items of this CTA (ring
  // stage g % STAGES; s_full / p_full complete once per tile), kact the items that have tiles
  // (q_full, q_empty, o_full, o_free complete once per such item).  Every role walks the same list.
  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tmap(&maps.q), prefetch_tmap(&maps.k), prefetch_tmap(&maps.v);
      if constexpr (DUAL) prefetch_tmap(&maps.tq), prefetch_tmap(&maps.tk), prefetch_tmap(&maps.tv);
      int g = 0, kact = 0;
      bool ok = true;
      FwdItem it;
      for (int k = 0; ok && k < k_max; ++k) {
        if (!get_item(k, it) || it.n_tiles == 0) continue;
        // The Q tiles are single-buffered: issuer A must be through with the previous item's.
        if (kact > 0 && !mbar_wait(q_empty, (kact - 1) & 1, ab, kAbortQFull)) break;
        mbar_expect_tx(q_full, C::N_Q * C::Q_BYTES);
        tma_load_4d(sQ, &maps.q, q_full, 0, it.m0, it.h, it.b);
        if constexpr (DUAL) tma_load_4d(sTQ, &maps.tq, q_full, 0, it.m0, it.h, it.b);
        LiveTiles live(it.live);
        for (int t = 0; t < it.n_tiles; ++t) {
          if constexpr (MK == 3)
            if (!live(t)) continue;
          const int st = g % STAGES;
          const uint32_t ph = (g / STAGES) & 1;
          if (!mbar_wait(kv_empty + st, ph ^ 1, ab, kAbortKvEmpty)) {
            ok = false;
            break;
          }
          unsigned char* base = sKV + st * (C::N_KV * C::KV_BYTES);
          mbar_expect_tx(kv_full + st, C::N_KV * C::KV_BYTES);
          const int n0 = t * BN;
          tma_load_4d(base + C::SLOT_K * C::KV_BYTES, &maps.k, kv_full + st, 0, n0, it.h, it.b);
          tma_load_4d(base + C::SLOT_V * C::KV_BYTES, &maps.v, kv_full + st, 0, n0, it.h, it.b);
          if constexpr (DUAL) {
            tma_load_4d(base + C::SLOT_TK * C::KV_BYTES, &maps.tk, kv_full + st, 0, n0, it.h, it.b);
            tma_load_4d(base + C::SLOT_TV * C::KV_BYTES, &maps.tv, kv_full + st, 0, n0, it.h, it.b);
          }
          ++g;
        }
        ++kact;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ issuer A: scores
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(Fmt<T>::kIdesc, BM, BN, 0, 0);       // 128 x 64
      constexpr uint32_t idesc_s2 = make_idesc(Fmt<T>::kIdesc, BM, 2 * BN, 0, 0);  // 128 x 128: [S | tS]
      const uint32_t aQ = smem_u32(sQ), aTQ = smem_u32(sTQ);
      int g = 0, kact = 0;
      bool ok = true;
      FwdItem it;
      for (int k = 0; ok && k < k_max; ++k) {
        if (!get_item(k, it) || it.n_tiles == 0) continue;
        if (!mbar_wait(q_full, kact & 1, ab, kAbortQFull)) break;
        LiveTiles live(it.live);
        for (int t = 0; t < it.n_tiles; ++t) {
          if constexpr (MK == 3)
            if (!live(t)) continue;
          const int st = g % STAGES;
          // S / tS still hold P / W of the previous tile (of this item or of the one before) until
          // issuer B's chain for it has completed.
          if (g > 0 && !mbar_wait(kv_empty + ((g - 1) % STAGES), ((g - 1) / STAGES) & 1, ab, kAbortKvEmpty)) {
            ok = false;
            break;
          }
          if (!mbar_wait(kv_full + st, (g / STAGES) & 1, ab, kAbortKvFull)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t aK = smem_u32(sKV + st * (C::N_KV * C::KV_BYTES)) + C::SLOT_K * C::KV_BYTES;
          if constexpr (DUAL) {
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks)  // [S | tS] = Q [K ; tK]^T
              umma_ss(tmem + C::COL_S, make_smem_desc(aQ + ks * 32, 16, 1024), make_smem_desc(aK + ks * 32, 16, 1024),
                      idesc_s2, ks > 0);
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks)  // tS += tQ K^T
              umma_ss(tmem + C::COL_TS, make_smem_desc(aTQ + ks * 32, 16, 1024), make_smem_desc(aK + ks * 32, 16, 1024),
                      idesc_s, 1);
          } else {
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks)
              umma_ss(tmem + C::COL_S, make_smem_desc(aQ + ks * 32, 16, 1024), make_smem_desc(aK + ks * 32, 16, 1024),
                      idesc_s, ks > 0);
          }
          tc_commit(s_full);
          ++g;
        }
        if (ok) tc_commit(q_empty);  // arrives when the item's last scores are complete
        ++kact;
      }
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------------ issuer B: outputs
    if (lane == 0) {
      constexpr uint32_t idesc_o = make_idesc(Fmt<T>::kIdesc, BM, D, 0, 1);       // 128 x 64, B MN-major
      constexpr uint32_t idesc_o2 = make_idesc(Fmt<T>::kIdesc, BM, 2 * D, 0, 1);  // 128 x 128: [O | tO']
      int g = 0, kact = 0;
      bool ok = true;
      FwdItem it;
      for (int k = 0; ok && k < k_max; ++k) {
        if (!get_item(k, it) || it.n_tiles == 0) continue;
        LiveTiles live(it.live);
        bool first = true;  // the item's first live tile
        for (int t = 0; t < it.n_tiles; ++t) {
          if constexpr (MK == 3)
            if (!live(t)) continue;
          const int st = g % STAGES;
          if (!mbar_wait(p_full, g & 1, ab, kAbortPFull)) {
            ok = false;
            break;
          }
          // The item's first tile overwrites O / tO': the previous item's epilogue must have read them.
          if constexpr (MK != 3) first = t == 0;
          if (first && kact > 0 && !mbar_wait(o_free, (kact - 1) & 1, ab, kAbortOFull)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t aV = smem_u32(sKV + st * (C::N_KV * C::KV_BYTES)) + C::SLOT_V * C::KV_BYTES;
          if constexpr (DUAL) {
#pragma unroll
            for (int kk = 0; kk < BN / 16; ++kk)  // [O | tO'] += P [V | tV]   (64-column chunks KV_BYTES apart)
              umma_ts(tmem + C::COL_O, tmem + C::COL_S + kk * 8, make_smem_desc(aV + kk * 2048, C::KV_BYTES, 1024),
                      idesc_o2, (!first || kk > 0));
#pragma unroll
            for (int kk = 0; kk < BN / 16; ++kk)  // tO' += W V
              umma_ts(tmem + C::COL_TO, tmem + C::COL_TS + kk * 8, make_smem_desc(aV + kk * 2048, C::KV_BYTES, 1024),
                      idesc_o, 1);
          } else {
#pragma unroll
            for (int kk = 0; kk < BN / 16; ++kk)
              umma_ts(tmem + C::COL_O, tmem + C::COL_S + kk * 8, make_smem_desc(aV + kk * 2048, C::KV_BYTES, 1024),
                      idesc_o, (!first || kk > 0));
          }
          tc_commit(kv_empty + st);
          first = false;
          ++g;
        }
        if (ok) tc_commit(o_full);
        ++kact;
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t tS = tmem + lane_off + C::COL_S, tTS = tmem + lane_off + C::COL_TS;
    const uint32_t tO = tmem + lane_off + C::COL_O, tTO = tmem + lane_off + C::COL_TO;
    const float scale_log2 = a.sm_scale * kLog2e;
    const float2 c2 = make_float2(scale_log2, scale_log2);
    const float2 sc2 = make_float2(a.sm_scale, a.sm_scale);
    bool alive = true;

    // Normalise and store one item's rows.  has_acc: the accumulators hold something (the item had
    // key tiles); then the item's last MMAs are waited for and O / tO' are released afterwards.
    auto epilogue = [&](int bh, int i, float m_used, float l_run, float mu_run, bool has_acc, int kact_of_item) -> bool {
      if (has_acc) {
        if (!mbar_wait(o_full, kact_of_item & 1, ab, kAbortOFull)) return false;
        tc_fence_after();
      }
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
        uint32_t ro[32], rt[DUAL ? 32 : 1];
        uint32_t po[16];
        if (has_acc) {
          tmem_ld32(tO + 32 * c, ro);
          if constexpr (DUAL) tmem_ld32(tTO + 32 * c, rt);
          tmem_wait_ld();
          if (c == D / 32 - 1) {  // everything is in registers: the accumulators may be overwritten
            tc_fence_before();
            mbar_arrive(o_free);
          }
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            ro[e] = 0u;
            if constexpr (DUAL) rt[e] = 0u;
          }
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
      return true;
    };

    int g = 0, kact = 0;
    FwdItem it;
    for (int k = 0; alive && k < k_max; ++k) {
      if (!get_item(k, it)) continue;
      const int i = it.m0 + row;
      if (it.n_tiles == 0) {  // no live key: zeros, lse = +inf
        alive = epilogue(it.bh, i, -INFINITY, 0.f, 0.f, false, 0);
        continue;
      }
      float m_used = -INFINITY, l_run = 0.f, mu_run = 0.f;
      // MK != 0: this thread's row of the mask / bias (rows past L are clamped; their results are not stored)
      constexpr bool BOOLM = MK == 1 || MK == 3;
      constexpr int MESZ = BOOLM ? 1 : 2;            // bytes per mask element
      constexpr int MW = MK == 0 ? 1 : 16 * MESZ;    // 32-bit words per row of a 64-key tile
      const unsigned char* mrow = nullptr;
      if constexpr (MK != 0)
        mrow = reinterpret_cast<const unsigned char*>(a.mask.ptr) +
               ((long long)it.b * a.mask.stride[0] + (long long)it.h * a.mask.stride[1] +
                (long long)min(i, L - 1) * a.mask.stride[2]) * MESZ;
      LiveTiles live(it.live);
      bool first = true;  // the item's first live tile
      for (int t = 0; t < it.n_tiles; ++t) {
        if constexpr (MK == 3)
          if (!live(t)) continue;
        const int n0 = t * BN;
        if constexpr (MK != 3) first = t == 0;
        uint32_t mw[MW];
        if constexpr (MK != 0) {  // issued before the wait: the loads fly while the scores are formed
#pragma unroll
          for (int j = 0; j < MW / 4; ++j) {
            uint4 r = make_uint4(0u, 0u, 0u, 0u);
            if (n0 + (j + 1) * (16 / MESZ) <= L) r = ldg_nc_v4(mrow + (size_t)n0 * MESZ + 16 * j);
            mw[4 * j] = r.x, mw[4 * j + 1] = r.y, mw[4 * j + 2] = r.z, mw[4 * j + 3] = r.w;
          }
        }
        if (!mbar_wait(s_full, g & 1, ab, kAbortSFull)) {
          alive = false;
          break;
        }
        tc_fence_after();
        uint32_t x0[32], x1[32];
        tmem_ld32(tS, x0);
        tmem_ld32(tS + 32, x1);
        tmem_wait_ld();
        // live key columns of this row inside the tile: col < col_hi
        int col_hi = min(BN, it.n_valid - n0);
        if (causal) col_hi = min(col_hi, i - n0 + 1);
        const bool partial = (n0 + BN > it.n_valid) || (causal && n0 + BN - 1 > it.m0);
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          float2 v0 = __fmul2_rn(ff2(x0[2 * c], x0[2 * c + 1]), c2);
          float2 v1 = __fmul2_rn(ff2(x1[2 * c], x1[2 * c + 1]), c2);
          if constexpr (BOOLM) {  // one byte per key: columns 2c, 2c+1 and 32+2c, 33+2c
            constexpr uint32_t kLoByte = 0xffu, kHiByte = 0xff00u;
            const uint32_t wa = mw[c >> 1] >> ((c & 1) * 16), wb = mw[8 + (c >> 1)] >> ((c & 1) * 16);
            if (!(wa & kLoByte)) v0.x = -INFINITY;
            if (!(wa & kHiByte)) v0.y = -INFINITY;
            if (!(wb & kLoByte)) v1.x = -INFINITY;
            if (!(wb & kHiByte)) v1.y = -INFINITY;
          }
          if constexpr (MK == 2) {  // scores are in log2 units: bias * log2(e)
            const float2 l2 = make_float2(kLog2e, kLog2e);
            v0 = __ffma2_rn(unpack2<T>(mw[c]), l2, v0);
            v1 = __ffma2_rn(unpack2<T>(mw[16 + c]), l2, v1);
          }
          if (partial) {
            if (2 * c >= col_hi) v0.x = -INFINITY;
            if (2 * c + 1 >= col_hi) v0.y = -INFINITY;
            if (32 + 2 * c >= col_hi) v1.x = -INFINITY;
            if (33 + 2 * c >= col_hi) v1.y = -INFINITY;
          }
          x0[2 * c] = __float_as_uint(v0.x), x0[2 * c + 1] = __float_as_uint(v0.y);
          x1[2 * c] = __float_as_uint(v1.x), x1[2 * c + 1] = __float_as_uint(v1.y);
          mx0 = fmaxf(mx0, v0.x), mx1 = fmaxf(mx1, v0.y), mx2 = fmaxf(mx2, v1.x), mx3 = fmaxf(mx3, v1.y);
        }
        const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
        // Lazy running max: keep the old reference while the new maximum is at most 2^8 above it.
        const bool grow = mx > m_used + 8.f;
        float alpha = 1.f;
        if (grow) {
          alpha = fast_exp2(m_used - mx);
          m_used = mx;
        }
        const float m_eff = (m_used == -INFINITY) ? 0.f : m_used;
        if (!first && __any_sync(0xffffffffu, grow)) {
          const float2 al2 = make_float2(alpha, alpha);
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t r[32];
            tmem_ld32(tO + 32 * c, r);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              const float2 v = __fmul2_rn(ff2(r[2 * e], r[2 * e + 1]), al2);
              r[2 * e] = __float_as_uint(v.x), r[2 * e + 1] = __float_as_uint(v.y);
            }
            tmem_st32(tO + 32 * c, r);
            if constexpr (DUAL) {
              tmem_ld32(tTO + 32 * c, r);
              tmem_wait_ld();
#pragma unroll
              for (int e = 0; e < 16; ++e) {
                const float2 v = __fmul2_rn(ff2(r[2 * e], r[2 * e + 1]), al2);
                r[2 * e] = __float_as_uint(v.x), r[2 * e + 1] = __float_as_uint(v.y);
              }
              tmem_st32(tTO + 32 * c, r);
            }
          }
        }
        const float2 nm2 = make_float2(-m_eff, -m_eff);
        float2 ls2a = make_float2(0.f, 0.f), ls2b = make_float2(0.f, 0.f);
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          const float2 e0 = __fadd2_rn(ff2(x0[2 * c], x0[2 * c + 1]), nm2);
          const float2 e1 = __fadd2_rn(ff2(x1[2 * c], x1[2 * c + 1]), nm2);
          const float2 p0 = make_float2(fast_exp2(e0.x), fast_exp2(e0.y));
          const float2 p1 = make_float2(fast_exp2(e1.x), fast_exp2(e1.y));
          x0[2 * c] = __float_as_uint(p0.x), x0[2 * c + 1] = __float_as_uint(p0.y);
          x1[2 * c] = __float_as_uint(p1.x), x1[2 * c + 1] = __float_as_uint(p1.y);
          ls2a = __fadd2_rn(ls2a, p0);
          ls2b = __fadd2_rn(ls2b, p1);
        }
        l_run = l_run * alpha + ((ls2a.x + ls2a.y) + (ls2b.x + ls2b.y));
        if constexpr (DUAL) {
          float2 ms2a = make_float2(0.f, 0.f), ms2b = make_float2(0.f, 0.f);
          uint32_t tt[32];
          uint32_t wp[16];
          tmem_ld32(tTS, tt);
          tmem_wait_ld();
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            const float2 w = __fmul2_rn(ff2(x0[2 * c], x0[2 * c + 1]), __fmul2_rn(ff2(tt[2 * c], tt[2 * c + 1]), sc2));
            ms2a = __fadd2_rn(ms2a, w);
            wp[c] = Elem<T>::pack(w.x, w.y);
          }
          tmem_ld32(tTS + 32, tt);  // second half is read before the first packed half is written below
          tmem_wait_ld();
          tmem_st16(tTS, wp);
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            const float2 w = __fmul2_rn(ff2(x1[2 * c], x1[2 * c + 1]), __fmul2_rn(ff2(tt[2 * c], tt[2 * c + 1]), sc2));
            ms2b = __fadd2_rn(ms2b, w);
            wp[c] = Elem<T>::pack(w.x, w.y);
          }
          tmem_st16(tTS + 16, wp);
          mu_run = mu_run * alpha + ((ms2a.x + ms2a.y) + (ms2b.x + ms2b.y));
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
        first = false;
        ++g;
      }
      if (!alive) break;
      // (Deferring this behind the softmax of the next item's first tile, as the backward does, was
      // measured slower here: the softmax warps are the critical path of this kernel.)
      if (!epilogue(it.bh, i, m_used, l_run, mu_run, true, kact)) break;
      ++kact;
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

static int fwd_sm_count() {
  static int cache[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (!cache[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    cache[dev] = n;
  }
  return cache[dev];
}

template <typename T, bool DUAL, int MK>
static int launch_fwd64(const jvpfa_fwd_args& a, cudaStream_t stream) {
  using C = Fwd64Cfg<DUAL>;
  int* status = tc5_status_device_ptr();
  if (!status) {
    set_last_cuda_error(cudaErrorUnknown, "status word address");
    return JVPFA_ERR_CUDA;
  }
  Fwd64Maps maps;
  const long long BH = (long long)a.B * a.H;
  const CUtensorMapDataType dt = Fmt<T>::kTma;
  // (64, L, H, B) maps: the inputs may be strided views (in_stride), e.g. (B,L,H,D) tensors seen as (B,H,L,D)
  const int64_t* st = a.in_stride;
  bool ok = encode_map4(&maps.q, dt, a.q, a.L, a.H, a.B, st, C::BM) && encode_map4(&maps.k, dt, a.k, a.L, a.H, a.B, st, C::BN) &&
            encode_map4(&maps.v, dt, a.v, a.L, a.H, a.B, st, C::BN);
  if (DUAL)
    ok = ok && encode_map4(&maps.tq, dt, a.tq, a.L, a.H, a.B, st, C::BM) &&
         encode_map4(&maps.tk, dt, a.tk, a.L, a.H, a.B, st, C::BN) && encode_map4(&maps.tv, dt, a.tv, a.L, a.H, a.B, st, C::BN);
  else
    maps.tq = maps.tk = maps.tv = maps.q;
  if (!ok) {
    set_last_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled(fwd d64)");
    return JVPFA_ERR_CUDA;
  }
  auto kern = fwd_tc5_d64_kernel<T, DUAL, MK>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
  if (e != cudaSuccess) {
    set_last_cuda_error(e, "cudaFuncSetAttribute(fwd_tc5_d64)");
    return JVPFA_ERR_CUDA;
  }
  const int sms = fwd_sm_count();
  if (sms <= 0) {
    set_last_cuda_error(cudaErrorUnknown, "multiprocessor count");
    return JVPFA_ERR_CUDA;
  }
  const long long n_items = (long long)((a.L + C::BM - 1) / C::BM) * BH;
  // Persistent CTAs (two per SM) pay off when the static list balances: causal shapes, where heavy and
  // light items alternate in every list, and uniform shapes whose item count fills the last round.
  // Otherwise (key padding: item lengths vary by batch; a thin last round) one CTA per item leaves the
  // balancing to the hardware scheduler; the kernel is the same, its list then has one entry.
  const long long slots = 2ll * sms;
  const long long rounds = (n_items + slots - 1) / slots;
  bool persistent = n_items > slots;
  if (persistent && a.mask.kind != JVPFA_MASK_CAUSAL)
    persistent = a.mask.kind != JVPFA_MASK_KVLEN ? (n_items * 100 >= rounds * slots * 95) : rounds >= 8;
  const int grid = (int)(persistent ? slots : n_items);
  kern<<<grid, C::NTHREADS, C::SMEM_BYTES, stream>>>(a, maps, status);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_cuda_error(e, "launch fwd_tc5_d64");
    return JVPFA_ERR_CUDA;
  }
  return JVPFA_OK;
}

}  // namespace tc5

template <typename T>
static int launch_fwd64_t(const jvpfa_fwd_args& a, cudaStream_t s) {
  const bool dual = a.tq != nullptr;
  if (a.mask.kind == JVPFA_MASK_BOOL && a.mask_tile_live != nullptr)
    return dual ? tc5::launch_fwd64<T, true, 3>(a, s) : tc5::launch_fwd64<T, false, 3>(a, s);
  if (a.mask.kind == JVPFA_MASK_BOOL)
    return dual ? tc5::launch_fwd64<T, true, 1>(a, s) : tc5::launch_fwd64<T, false, 1>(a, s);
  if (a.mask.kind == JVPFA_MASK_BIAS)
    return dual ? tc5::launch_fwd64<T, true, 2>(a, s) : tc5::launch_fwd64<T, false, 2>(a, s);
  if (!dual) return launch_fwd_tc5_sub32(a, s);  // primal only: 32-key sub-tile pipeline (fwd_tc5_sub32.cu)
  return tc5::launch_fwd64<T, true, 0>(a, s);
}

int launch_fwd_tc5_d64(const jvpfa_fwd_args& a, cudaStream_t s) {
  return a.dtype == JVPFA_BF16 ? launch_fwd64_t<__nv_bfloat16>(a, s) : launch_fwd64_t<__half>(a, s);
}

}  // namespace jvpfa
