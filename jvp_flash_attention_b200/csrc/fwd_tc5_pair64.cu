// Fused primal (+ tangent) attention forward for head dimension 64 (bf16 / fp16) on tcgen05 / TMA /
// TMEM, organised so that the softmax never sits between two dependent MMAs of the same tile.
//
// One CTA per SM owns a PAIR of 128-row query tiles (256 query rows of one (batch, head)) and walks a
// static list of such pairs.  The two query tiles are two independent pipelines that share every
// K / tK / V / tV stage brought in by TMA (so each key tile is fetched once per 256 query rows):
//
//   issuer X (one thread per query tile):   [S | tS] = Q [K ; tK]^T (N=128) ; tS += tQ K^T (N=64)   -> s_full[X]
//                                           [O | tO'] += P [V | tV] (N=128) ; tO' += W V   (N=64)   -> pv_done[X], kv_empty
//   softmax X (one warpgroup per query tile, thread <-> query row <-> TMEM lane)
//
// P and W = P * tS * scale leave the softmax threads through SHARED memory (128-byte-swizzled K-major
// tiles, the layout TMA gives Q), not through TMEM.  The score accumulators are therefore free as soon
// as the softmax threads have copied them to registers (s_free[X]), and the issuer forms the scores of
// key tile j+1 while the softmax of tile j is still computing:
//
//   issue order per query tile:   S(0) ; S(1) PV(0) ; S(2) PV(1) ; ... ; PV(last)
//
// TMEM columns per query tile: S [64] | tS [64] | O [64] | tO' [64]; two query tiles = 512 columns.
// Online softmax with lazy rescaling: the running reference maximum is raised only when the tile maximum
// exceeds it by more than 2^8, and only then are O / tO' rescaled in TMEM (after PV of the previous tile
// has completed).  Row arithmetic uses packed fp32x2 instructions.
//
// Masks (template parameter MK): 0 = none / causal / key padding by index comparison; 1 = uint8 mask;
// 2 = additive bias of the element type; 3 = uint8 mask with the tile bitmap written by jvpfa_mask_tiles
// (one bit per 128-query x 64-key tile).  A softmax thread owns one query row, so its share of a mask tile
// is 64 consecutive elements, fetched as 16-byte read-only loads before the thread waits for the scores.
// With a bitmap the two query tiles may need different key tiles: the producer loads the union, and an
// issuer that does not use a loaded tile only releases it.
#include "tc5_common.cuh"

namespace jvpfa {
namespace tc5 {

template <bool DUAL>
struct FwdPairCfg {
  static constexpr int D = 64;
  static constexpr int BM = 128;  // rows of one query tile
  static constexpr int NQ = 2;    // query tiles per CTA
  static constexpr int BN = 64;
  static constexpr int STAGES = 3;
  static constexpr int NTHREADS = 384;  // warpgroup 0: TMA producer, two issuers, one idle warp; warpgroups 1, 2: softmax
  static constexpr int Q_BYTES = BM * D * 2;   // 16 KiB
  static constexpr int KV_BYTES = BN * D * 2;  // 8 KiB
  static constexpr int P_BYTES = BM * BN * 2;  // 16 KiB
  static constexpr int N_QT = DUAL ? 2 : 1;    // Q, tQ
  static constexpr int N_KV = DUAL ? 4 : 2;    // K, tK, V, tV
  static constexpr int N_P = DUAL ? 2 : 1;     // P, W
  static constexpr int SLOT_K = 0, SLOT_TK = 1, SLOT_V = DUAL ? 2 : 1, SLOT_TV = 3;
  static constexpr int STAGE_BYTES = N_KV * KV_BYTES;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_KV = NQ * N_QT * Q_BYTES;
  static constexpr int OFF_P = OFF_KV + STAGES * STAGE_BYTES;
  static constexpr int TILE_BYTES = OFF_P + NQ * N_P * P_BYTES;
  static constexpr int SMEM_BYTES = TILE_BYTES + 256 + 1024;
  static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
  static constexpr int COL_S = 0;
  static constexpr int COL_TS = 64;
  static constexpr int COL_O = DUAL ? 128 : 64;
  static constexpr int COL_TO = 192;
  // Primal only: half of the columns are free, so P (packed 16-bit, 32 columns) stays in TMEM in a place of its
  // own and feeds the output MMAs as their A operand; nothing of P touches shared memory.
  static constexpr int COL_P = 128;
  static constexpr int COLS_PER_Q = 256;
  static constexpr int COLS_ALLOC = NQ * COLS_PER_Q;
};

struct FwdPairMaps {
  CUtensorMap q, tq, k, tk, v, tv;
  CUtensorMap o, to;  // outputs, stored tile-wise from shared memory
};

// TMA store of one (64 x rows) tile from shared memory; rows past the tensor's extent are not written.
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, const void* smem_src, int x, int y, int z, int w) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(map),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z), "r"(w)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }



__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// Makes this thread's shared-memory writes visible to the async proxy (the tensor core reads operands through it).
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// One work item: two neighbouring 128-row query tiles of one (batch, head).  Per-query-tile fields are plain
// scalars picked with a select (arrays indexed by the query tile would live in local memory).
struct PairItem {
  int bh, b, h, m0, n_valid;
  int nt0, nt1;      // key tiles in range of each query tile (0: the tile has no row or no key)
  int last0, last1;  // index of the last key tile each query tile uses, -1 when it uses none
  int n_load;        // key tiles to walk: max(nt0, nt1)
  const unsigned long long *live0, *live1;  // MK == 3: the query tiles' words of the tile bitmap
  __device__ __forceinline__ int nt(int x) const { return x ? nt1 : nt0; }
  __device__ __forceinline__ int last(int x) const { return x ? last1 : last0; }
};

// Walks an item's key tiles in order: bit X of the result says that query tile X uses tile j.
template <int MK>
struct TileUse {
  const int nt0, nt1;
  const unsigned long long *l0, *l1;
  unsigned long long w0, w1;
  __device__ __forceinline__ explicit TileUse(const PairItem& i)
      : nt0(i.nt0), nt1(i.nt1), l0(i.live0), l1(i.live1), w0(0ull), w1(0ull) {}
  __device__ __forceinline__ int operator()(int j) {
    int m = (j < nt0 ? 1 : 0) | (j < nt1 ? 2 : 0);
    if constexpr (MK == 3) {
      if ((j & 63) == 0) {
        w0 = __ldg(l0 + (j >> 6));
        w1 = __ldg(l1 + (j >> 6));
      }
      m &= (int)((w0 >> (j & 63)) & 1ull) | ((int)((w1 >> (j & 63)) & 1ull) << 1);
    }
    return m;
  }
};

template <typename T, bool DUAL, int MK>
__global__ void __launch_bounds__(384, 1)
fwd_tc5_pair64_kernel(const jvpfa_fwd_args a, const __grid_constant__ FwdPairMaps maps, int* status) {
  using C = FwdPairCfg<DUAL>;
  constexpr int D = 64, BM = C::BM, BN = C::BN, STAGES = C::STAGES;

  const bool dead_on_entry = *(volatile int*)status != 0;  // an earlier bounded wait gave up

  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  unsigned char* smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  unsigned char* sQ = smem + C::OFF_Q;    // [query tile][Q, tQ]
  unsigned char* sKV = smem + C::OFF_KV;  // [stage][K, tK, V, tV]
  unsigned char* sP = smem + C::OFF_P;    // [query tile][P, W]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::TILE_BYTES);
  uint64_t* q_full = bars + 0;
  uint64_t* q_empty = bars + 1;   // both issuers are through with the item's Q tiles
  uint64_t* kv_full = bars + 2;   // [STAGES]
  uint64_t* kv_empty = kv_full + STAGES;  // [STAGES], one arrival per issuer
  uint64_t* s_full = kv_empty + STAGES;   // [2] per query tile from here on
  uint64_t* s_free = s_full + 2;          // the softmax threads hold the scores in registers
  uint64_t* p_full = s_free + 2;          // P / W are in shared memory
  uint64_t* pv_done = p_full + 2;         // the tile's output MMAs are complete
  uint64_t* o_free = pv_done + 2;         // the epilogue has read the item's accumulators
  uint64_t* wg_bar = o_free + 2;          // meeting point of a softmax warpgroup's 128 threads (bounded, unlike bar.sync)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(wg_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int L = a.L;
  const int BH = a.B * a.H;
  const bool causal = a.mask.kind == JVPFA_MASK_CAUSAL;
  const int n_q_tiles = (L + BM - 1) / BM;
  const int n_pairs = (n_q_tiles + 1) / 2;
  const int n_items = n_pairs * BH;
  const int G = (int)gridDim.x, cta = (int)blockIdx.x;
  const int k_max = (n_items + G - 1) / G;

  // Item k of this CTA: items are ranked heaviest first (for causal masks the last pair is the longest) and
  // dealt in serpentine order.
  auto get_item = [&](int k, PairItem& it) -> bool {
    const int w = k * G + ((k & 1) ? (G - 1 - cta) : cta);
    if (w >= n_items) return false;
    int pair;
    if (causal) {
      const int rank = w / BH;
      it.bh = w - rank * BH;
      pair = n_pairs - 1 - rank;
    } else {  // equal weights: the pairs of a head run side by side and share its K / V in L2
      it.bh = w / n_pairs;
      pair = w - it.bh * n_pairs;
    }
    it.m0 = pair * (2 * BM);
    it.b = it.bh / a.H;
    it.h = it.bh - it.b * a.H;
    it.n_valid = L;
    if (a.mask.kind == JVPFA_MASK_KVLEN) {
      const int n = a.mask.kv_len[it.b];
      it.n_valid = n < 0 ? 0 : (n > L ? L : n);
    }
    {
      int e0 = it.m0 < L ? it.n_valid : 0, e1 = it.m0 + BM < L ? it.n_valid : 0;
      if (causal) e0 = min(e0, it.m0 + BM), e1 = min(e1, it.m0 + 2 * BM);
      it.nt0 = (e0 + BN - 1) / BN, it.nt1 = (e1 + BN - 1) / BN;
      it.last0 = it.nt0 - 1, it.last1 = it.nt1 - 1;
      it.live0 = it.live1 = nullptr;
    }
    if constexpr (MK == 3) {
      // the bitmap has the mask's own extents: broadcast dimensions (stride 0) have one entry
      const int n_words = ((L + BN - 1) / BN + 63) >> 6;
      const long long hm = (a.mask.stride[0] ? (long long)it.b * (a.mask.stride[1] ? a.H : 1) : 0) +
                           (a.mask.stride[1] ? it.h : 0);
      auto scan = [&](int x, int& nt, int& last, const unsigned long long*& live) {
        const int qt = min(it.m0 / BM + x, n_q_tiles - 1);
        const long long qm = a.mask.stride[2] ? hm * n_q_tiles + qt : hm;
        live = reinterpret_cast<const unsigned long long*>(a.mask_tile_live) + qm * n_words;
        last = -1;
        for (int w2 = 0; w2 < (nt + 63) >> 6; ++w2) {
          unsigned long long bits = __ldg(live + w2);
          const int rem = nt - 64 * w2;
          if (rem < 64) bits &= (1ull << rem) - 1ull;
          if (bits) last = 64 * w2 + 63 - __clzll(bits);
        }
        if (last < 0) nt = 0;  // nothing to attend to: zeros and lse = +inf, as for kv_len = 0
      };
      scan(0, it.nt0, it.last0, it.live0);
      scan(1, it.nt1, it.last1, it.live1);
    }
    it.n_load = max(it.nt0, it.nt1);
    return true;
  };

  // lse = NaN for every row of this CTA's items: the results of this launch are not to be trusted
  auto poison = [&]() {
    PairItem it;
    for (int k = 0; k < k_max; ++k) {
      if (!get_item(k, it)) continue;
      const int i = it.m0 + tid;
      if (tid < 2 * BM && i < L) a.lse[(size_t)it.bh * L + i] = poison_f32();
    }
  };
  if (dead_on_entry) {
    poison();
    return;
  }

  if (tid == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 2);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(kv_full + s, 1);
      mbar_init(kv_empty + s, 2);
    }
    for (int x = 0; x < 2; ++x) {
      mbar_init(s_full + x, 1);
      mbar_init(s_free + x, 128);
      mbar_init(p_full + x, 128);
      mbar_init(pv_done + x, 1);
      mbar_init(o_free + x, 128);
      mbar_init(wg_bar + x, 128);
    }
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

  // Phase counters, kept alike by every role: g counts the key tiles loaded by this CTA (ring stage g % STAGES),
  // kact the items that load anything (q_full / q_empty), t[X] the key tiles query tile X has used (s_full,
  // s_free, p_full, pv_done of X complete once per such tile), kx[X] the items in which X used a tile (o_free).
  // The four warps of warpgroup 0 need few registers; the softmax threads hold two score tiles each.
  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 80;");
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
  }
  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tmap(&maps.q), prefetch_tmap(&maps.k), prefetch_tmap(&maps.v);
      if constexpr (DUAL) prefetch_tmap(&maps.tq), prefetch_tmap(&maps.tk), prefetch_tmap(&maps.tv);
      int g = 0, kact = 0;
      bool ok = true;
      PairItem it;
      for (int k = 0; ok && k < k_max; ++k) {
        if (!get_item(k, it) || it.n_load == 0) continue;
        // The Q tiles are single-buffered: both issuers must be through with the previous item's.
        if (kact > 0 && !mbar_wait(q_empty, (kact - 1) & 1, ab, kAbortQFull)) break;
        mbar_expect_tx(q_full, C::NQ * C::N_QT * C::Q_BYTES);
#pragma unroll
        for (int x = 0; x < 2; ++x) {  // a tile that starts past L reads as zeros
          unsigned char* dst = sQ + x * C::N_QT * C::Q_BYTES;
          tma_load_4d(dst, &maps.q, q_full, 0, it.m0 + x * BM, it.h, it.b);
          if constexpr (DUAL) tma_load_4d(dst + C::Q_BYTES, &maps.tq, q_full, 0, it.m0 + x * BM, it.h, it.b);
        }
        TileUse<MK> use(it);
        for (int j = 0; j < it.n_load; ++j) {
          if (use(j) == 0) continue;
          const int st = g % STAGES;
          if (!mbar_wait(kv_empty + st, ((g / STAGES) & 1) ^ 1, ab, kAbortKvEmpty)) {
            ok = false;
            break;
          }
          unsigned char* base = sKV + st * C::STAGE_BYTES;
          mbar_expect_tx(kv_full + st, C::STAGE_BYTES);
          const int n0 = j * BN;
          tma_load_4d(base + C::SLOT_K * C::KV_BYTES, &maps.k, kv_full + st, 0, n0, it.h, it.b);
          if constexpr (DUAL) tma_load_4d(base + C::SLOT_TK * C::KV_BYTES, &maps.tk, kv_full + st, 0, n0, it.h, it.b);
          tma_load_4d(base + C::SLOT_V * C::KV_BYTES, &maps.v, kv_full + st, 0, n0, it.h, it.b);
          if constexpr (DUAL) tma_load_4d(base + C::SLOT_TV * C::KV_BYTES, &maps.tv, kv_full + st, 0, n0, it.h, it.b);
          ++g;
        }
        ++kact;
      }
    }
  } else if (warp <= 2) {
    // ------------------------------------------------------------------ issuer of query tile X
    // One thread.  Whatever it executes between two MMAs is pure latency for the tensor pipe, so stage and
    // barrier cursors, parities and the low words of the operand descriptors live in registers and advance by
    // additions (descriptor = constant high word kDescHi + (byte address >> 4) in the low word).
    if (lane == 0) {
      const int X = warp - 1;
      constexpr uint32_t idesc_s = make_idesc(Fmt<T>::kIdesc, BM, BN, 0, 0);       // 128 x 64
      constexpr uint32_t idesc_s2 = make_idesc(Fmt<T>::kIdesc, BM, 2 * BN, 0, 0);  // 128 x 128: [S | tS]
      constexpr uint32_t idesc_o = make_idesc(Fmt<T>::kIdesc, BM, D, 0, 1);        // 128 x 64, B MN-major
      constexpr uint32_t idesc_o2 = make_idesc(Fmt<T>::kIdesc, BM, 2 * D, 0, 1);   // 128 x 128: [O | tO']
      constexpr uint32_t kLoV = (uint32_t)(C::KV_BYTES >> 4) << 16;  // [V | tV]: 64-column chunks KV_BYTES apart
      constexpr uint32_t STAGE16 = C::STAGE_BYTES >> 4;
      const uint32_t q_lo = kDescLo | (smem_u32(sQ + X * C::N_QT * C::Q_BYTES) >> 4), tq_lo = q_lo + (C::Q_BYTES >> 4);
      const uint32_t p_lo = kDescLo | (smem_u32(sP + X * C::N_P * C::P_BYTES) >> 4), w_lo = p_lo + (C::P_BYTES >> 4);
      const uint32_t k_lo0 = kDescLo | ((smem_u32(sKV) + C::SLOT_K * C::KV_BYTES) >> 4);
      const uint32_t v_lo0 = kLoV | ((smem_u32(sKV) + C::SLOT_V * C::KV_BYTES) >> 4);
      const uint32_t bar_kv_full = smem_u32(kv_full), bar_kv_empty = smem_u32(kv_empty);
      const uint32_t bar_s_full = smem_u32(s_full + X), bar_s_free = smem_u32(s_free + X);
      const uint32_t bar_p_full = smem_u32(p_full + X), bar_pv_done = smem_u32(pv_done + X);
      const uint32_t bar_o_free = smem_u32(o_free + X), bar_q_empty = smem_u32(q_empty);
      const uint32_t tq = tmem + X * C::COLS_PER_Q;
      uint32_t st = 0, st_par = 0;  // ring stage of the next loaded tile and the parity of its kv_full phase
      uint32_t tpar = 0;            // parity of the phase that this query tile's next used tile completes
      bool any_t = false;           // this query tile has used a tile before
      int kact = 0, kx = 0;
      bool ok = true;
      PairItem it;

      // [O | tO'] (+)= P [V | tV] ; tO' += W V for the tile in ring stage pst, whose phases have parity ppar
      auto issue_pv = [&](uint32_t pst, uint32_t ppar, bool first) -> bool {
        if (!mbar_wait_u32(bar_p_full, ppar, ab, kAbortPFull)) return false;
        // The item's first tile overwrites O / tO': the previous item's epilogue must have read them.
        if (first && kx > 0 && !mbar_wait_u32(bar_o_free, (kx - 1) & 1, ab, kAbortOFull)) return false;
        tc_fence_after();
        const uint32_t v_lo = v_lo0 + pst * STAGE16;
        if constexpr (DUAL) {
          umma_ss_lo_dyn(tq + C::COL_O, p_lo, v_lo, idesc_o2, first ? 0u : 1u);
#pragma unroll
          for (int kk = 1; kk < BN / 16; ++kk) umma_ss_lo<true>(tq + C::COL_O, p_lo + kk * 2, v_lo + kk * 128, idesc_o2);
#pragma unroll
          for (int kk = 0; kk < BN / 16; ++kk) umma_ss_lo<true>(tq + C::COL_TO, w_lo + kk * 2, v_lo + kk * 128, idesc_o);
        } else {  // P from TMEM
          umma_ts_lo_dyn(tq + C::COL_O, tq + C::COL_P, v_lo, idesc_o, first ? 0u : 1u);
#pragma unroll
          for (int kk = 1; kk < BN / 16; ++kk) umma_ts_lo<true>(tq + C::COL_O, tq + C::COL_P + kk * 8, v_lo + kk * 128, idesc_o);
        }
        tc_commit_u32(bar_kv_empty + 8 * pst);
        tc_commit_u32(bar_pv_done);
        return true;
      };

      for (int k = 0; ok && k < k_max; ++k) {
        if (!get_item(k, it) || it.n_load == 0) continue;
        // waited for by both issuers in every item, used or not: a parity wait must see every phase
        if (!mbar_wait(q_full, kact & 1, ab, kAbortQFull)) break;
        const int my_last = it.last(X);
        bool pend = false, pend_first = false, first = true;
        uint32_t pend_st = 0, pend_par = 0;
        TileUse<MK> use(it);
        for (int j = 0; j < it.n_load; ++j) {
          const int m = use(j);
          if (m == 0) continue;
          if (!mbar_wait_u32(bar_kv_full + 8 * st, st_par, ab, kAbortKvFull)) {
            ok = false;
            break;
          }
          if (m & (1 << X)) {
            // S / tS of the previous tile (of this item or the one before) must be in the softmax threads' registers
            if (any_t && !mbar_wait_u32(bar_s_free, tpar ^ 1, ab, kAbortSFull)) {
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t k_lo = k_lo0 + st * STAGE16;
            if constexpr (DUAL) {
              umma_ss_lo<false>(tq + C::COL_S, q_lo, k_lo, idesc_s2);  // [S | tS] = Q [K ; tK]^T
#pragma unroll
              for (int ks = 1; ks < D / 16; ++ks) umma_ss_lo<true>(tq + C::COL_S, q_lo + ks * 2, k_lo + ks * 2, idesc_s2);
#pragma unroll
              for (int ks = 0; ks < D / 16; ++ks) umma_ss_lo<true>(tq + C::COL_TS, tq_lo + ks * 2, k_lo + ks * 2, idesc_s);  // tS += tQ K^T
            } else {
              umma_ss_lo<false>(tq + C::COL_S, q_lo, k_lo, idesc_s);
#pragma unroll
              for (int ks = 1; ks < D / 16; ++ks) umma_ss_lo<true>(tq + C::COL_S, q_lo + ks * 2, k_lo + ks * 2, idesc_s);
            }
            tc_commit_u32(bar_s_full);
            if (j == my_last) tc_commit_u32(bar_q_empty);  // arrives when the item's last scores are complete
            if (pend && !issue_pv(pend_st, pend_par, pend_first)) {
              ok = false;
              break;
            }
            pend = true, pend_st = st, pend_par = tpar, pend_first = first, first = false;
            tpar ^= 1, any_t = true;
          } else {
            // Loaded for the other query tile only.  A pending output product holds an older ring stage: it goes
            // out first, or the producer could wait for that stage while this thread waits for the producer.
            if (pend) {
              if (!issue_pv(pend_st, pend_par, pend_first)) {
                ok = false;
                break;
              }
              pend = false;
            }
            mbar_arrive(kv_empty + st);
          }
          if (++st == STAGES) st = 0, st_par ^= 1;
        }
        if (!ok) break;
        if (pend && !issue_pv(pend_st, pend_par, pend_first)) break;
        if (!first)
          ++kx;  // this query tile used key tiles in the item (its q_empty arrival went out with the last scores)
        else
          mbar_arrive(q_empty);
        ++kact;
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ softmax + epilogue of query tile X
    const int X = (warp - 4) >> 2;
    const int quarter = warp & 3;  // the TMEM lane quarter this warp may access
    const int row = quarter * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t tq = tmem + lane_off + X * C::COLS_PER_Q;
    const uint32_t tS = tq + C::COL_S, tTS = tq + C::COL_TS, tO = tq + C::COL_O, tTO = tq + C::COL_TO;
    // this thread's row of the P / W tiles: 16-byte chunk c sits at position c ^ (row & 7) of the 128-byte row
    const uint32_t pP = smem_u32(sP + X * C::N_P * C::P_BYTES) + row * 128, pW = pP + C::P_BYTES;
    const uint32_t sw = (uint32_t)(row & 7);
    const float scale_log2 = a.sm_scale * kLog2e;
    const float2 c2 = make_float2(scale_log2, scale_log2);
    const float2 sc2 = make_float2(a.sm_scale, a.sm_scale);
    bool alive = true;
    int kx = 0;
    uint32_t t = 0;

    // The item's O / tO rows leave through the query tile's P / W buffers (idle between items) and one TMA store
    // per output, issued by the warpgroup's first thread.  Before anybody writes those buffers again the store
    // must have read them: release_staging().
    bool store_pending = false;
    uint32_t wg_phase = 0;
    auto wg_sync = [&]() -> bool {
      mbar_arrive(wg_bar + X);
      const bool ok = mbar_wait(wg_bar + X, wg_phase & 1, ab, kAbortAux);
      ++wg_phase;
      return ok;
    };
    auto release_staging = [&]() -> bool {
      if (!store_pending) return true;
      store_pending = false;
      if (row == 0) tma_store_wait_read();
      return wg_sync();
    };
    // Normalise and store one item's rows.  has_acc: the accumulators hold something (the query tile used key
    // tiles); then the last tile's output MMAs are waited for and O / tO' are released afterwards.
    auto epilogue = [&](const PairItem& it, int i, float m_used, float l_run, float mu_run, bool has_acc) -> bool {
      if (has_acc) {
        if (!mbar_wait(pv_done + X, (t - 1) & 1, ab, kAbortOFull)) return false;
        tc_fence_after();
      }
      if (!release_staging()) return false;
      const bool empty = !(l_run > 0.f);
      const float inv_l = empty ? 0.f : 1.f / l_run;
      const float mu_n = mu_run * inv_l;
      if (i < L) {
        a.lse[(size_t)it.bh * L + i] = empty ? INFINITY : (m_used + log2f(l_run));
        if constexpr (DUAL) a.mu[(size_t)it.bh * L + i] = mu_n;
      }
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
            mbar_arrive(o_free + X);
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
#pragma unroll
        for (int e = 0; e < 4; ++e)
          st_shared_v4(pP + (((uint32_t)(4 * c + e) ^ sw) << 4), po[4 * e], po[4 * e + 1], po[4 * e + 2], po[4 * e + 3]);
        if constexpr (DUAL) {
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const float t0 = __uint_as_float(rt[2 * e]) * inv_l - mu_n * __uint_as_float(ro[2 * e]);
            const float t1 = __uint_as_float(rt[2 * e + 1]) * inv_l - mu_n * __uint_as_float(ro[2 * e + 1]);
            po[e] = Elem<T>::pack(t0, t1);
          }
#pragma unroll
          for (int e = 0; e < 4; ++e)
            st_shared_v4(pW + (((uint32_t)(4 * c + e) ^ sw) << 4), po[4 * e], po[4 * e + 1], po[4 * e + 2], po[4 * e + 3]);
        }
      }
      fence_proxy_async_smem();
      if (!wg_sync()) return false;
      const int mX = it.m0 + X * BM;
      if (row == 0 && mX < L) {
        tma_store_4d(&maps.o, sP + X * C::N_P * C::P_BYTES, 0, mX, it.h, it.b);
        if constexpr (DUAL) tma_store_4d(&maps.to, sP + X * C::N_P * C::P_BYTES + C::P_BYTES, 0, mX, it.h, it.b);
        tma_store_commit();
      }
      store_pending = true;
      return true;
    };

    PairItem it;
    for (int k = 0; alive && k < k_max; ++k) {
      if (!get_item(k, it)) continue;
      const int mX = it.m0 + X * BM;
      const int i = mX + row;
      if (it.last(X) < 0) {  // no live key for this query tile: zeros, lse = +inf
        alive = epilogue(it, i, -INFINITY, 0.f, 0.f, false);
        continue;
      }
      float m_used = -INFINITY, l_run = 0.f, mu_run = 0.f;
      // MK != 0: this thread's row of the mask / bias (rows past L are clamped; their results are not stored)
      constexpr bool BOOLM = MK == 1 || MK == 3;
      constexpr int MESZ = BOOLM ? 1 : 2;          // bytes per mask element
      constexpr int MW = MK == 0 ? 1 : 16 * MESZ;  // 32-bit words per row of a 64-key tile
      // The tangent scores are fetched together with the scores, so that the accumulators are free at once,
      // where the registers allow it (no mask words to hold).
      constexpr bool EARLY_TS = DUAL && MK == 0;
      const unsigned char* mrow = nullptr;
      if constexpr (MK != 0)
        mrow = reinterpret_cast<const unsigned char*>(a.mask.ptr) +
               ((long long)it.b * a.mask.stride[0] + (long long)it.h * a.mask.stride[1] +
                (long long)min(i, L - 1) * a.mask.stride[2]) * MESZ;
      TileUse<MK> use(it);
      bool first = true;  // the item's first tile used by this query tile
      for (int j = 0; j < it.n_load; ++j) {
        if (!(use(j) & (1 << X))) continue;
        const int n0 = j * BN;
        uint32_t mw[MW];
        if constexpr (MK != 0) {  // issued before the wait: the loads fly while the scores are formed
#pragma unroll
          for (int q4 = 0; q4 < MW / 4; ++q4) {
            uint4 r = make_uint4(0u, 0u, 0u, 0u);
            if (n0 + (q4 + 1) * (16 / MESZ) <= L) r = ldg_nc_v4(mrow + (size_t)n0 * MESZ + 16 * q4);
            mw[4 * q4] = r.x, mw[4 * q4 + 1] = r.y, mw[4 * q4 + 2] = r.z, mw[4 * q4 + 3] = r.w;
          }
        }
        if (!mbar_wait(s_full + X, t & 1, ab, kAbortSFull)) {
          alive = false;
          break;
        }
        tc_fence_after();
        uint32_t x0[32], x1[32];
        uint32_t t0[EARLY_TS ? 32 : 1], t1[EARLY_TS ? 32 : 1];
        tmem_ld32(tS, x0);
        tmem_ld32(tS + 32, x1);
        if constexpr (EARLY_TS) {
          tmem_ld32(tTS, t0);
          tmem_ld32(tTS + 32, t1);
        }
        tmem_wait_ld();
        if constexpr (EARLY_TS || !DUAL) {
          tc_fence_before();
          mbar_arrive(s_free + X);
        }
        // live key columns of this row inside the tile: col < col_hi
        int col_hi = min(BN, it.n_valid - n0);
        if (causal) col_hi = min(col_hi, i - n0 + 1);
        const bool partial = (n0 + BN > it.n_valid) || (causal && n0 + BN - 1 > mX);
        // Row maximum of the tile in log2 units.  Without a mask or bias it is taken over the raw scores (the scale
        // is positive) and the scaling is folded into the exponent's multiply-add; otherwise the scores are scaled,
        // biased and masked first.
        float mx;
        if constexpr (MK == 0) {
          if (partial) {
#pragma unroll
            for (int c = 0; c < 32; ++c) {
              if (c >= col_hi) x0[c] = 0xff800000u;  // -inf
              if (32 + c >= col_hi) x1[c] = 0xff800000u;
            }
          }
          float mxa = -INFINITY, mxb = -INFINITY, mxc = -INFINITY, mxd = -INFINITY;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            mxa = max3(mxa, __uint_as_float(x0[4 * c]), __uint_as_float(x0[4 * c + 1]));
            mxb = max3(mxb, __uint_as_float(x0[4 * c + 2]), __uint_as_float(x0[4 * c + 3]));
            mxc = max3(mxc, __uint_as_float(x1[4 * c]), __uint_as_float(x1[4 * c + 1]));
            mxd = max3(mxd, __uint_as_float(x1[4 * c + 2]), __uint_as_float(x1[4 * c + 3]));
          }
          mx = max3(mxa, mxb, fmaxf(mxc, mxd)) * scale_log2;
        } else {
          float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            float2 v0 = __fmul2_rn(pf2(x0[2 * c], x0[2 * c + 1]), c2);
            float2 v1 = __fmul2_rn(pf2(x1[2 * c], x1[2 * c + 1]), c2);
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
          mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
        }
        // Lazy running max: keep the old reference while the new maximum is at most 2^8 above it.
        const bool grow = mx > m_used + 8.f;
        float alpha = 1.f;
        if (grow) {
          alpha = fast_exp2(m_used - mx);
          m_used = mx;
        }
        const float m_eff = (m_used == -INFINITY) ? 0.f : m_used;
        bool prev_pv_seen = false;  // the previous tile's output MMAs are known to be complete
        if (!first && __any_sync(0xffffffffu, grow)) {
          // O / tO' are rescaled in place: the previous tile's output MMAs must have landed
          if (!mbar_wait(pv_done + X, (t - 1) & 1, ab, kAbortOFull)) {
            alive = false;
            break;
          }
          prev_pv_seen = true;
          tc_fence_after();
          const float2 al2 = make_float2(alpha, alpha);
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t r[32];
            tmem_ld32(tO + 32 * c, r);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              const float2 v = __fmul2_rn(pf2(r[2 * e], r[2 * e + 1]), al2);
              r[2 * e] = __float_as_uint(v.x), r[2 * e + 1] = __float_as_uint(v.y);
            }
            tmem_st32(tO + 32 * c, r);
            if constexpr (DUAL) {
              tmem_ld32(tTO + 32 * c, r);
              tmem_wait_ld();
#pragma unroll
              for (int e = 0; e < 16; ++e) {
                const float2 v = __fmul2_rn(pf2(r[2 * e], r[2 * e + 1]), al2);
                r[2 * e] = __float_as_uint(v.x), r[2 * e + 1] = __float_as_uint(v.y);
              }
              tmem_st32(tTO + 32 * c, r);
            }
          }
          tmem_wait_st();
        }
        // Exponentials, row sums, W = P * tS * scale and the packing to 16 bit in one loop per half tile, so that
        // the special-function unit's latency is covered by the arithmetic of the neighbouring columns.
        const float2 nm2 = make_float2(-m_eff, -m_eff);
        float2 ls2 = make_float2(0.f, 0.f), ms2 = make_float2(0.f, 0.f);
        uint32_t pp[32], wp[DUAL ? 32 : 1];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          uint32_t* xs = hh ? x1 : x0;
          uint32_t tt[(DUAL && !EARLY_TS) ? 32 : 1];
          if constexpr (DUAL && !EARLY_TS) {
            tmem_ld32(tTS + 32 * hh, tt);
            tmem_wait_ld();
            if (hh == 1) {
              tc_fence_before();
              mbar_arrive(s_free + X);  // both score accumulators are in registers now
            }
          }
          const uint32_t* ts = EARLY_TS ? (hh ? t1 : t0) : tt;
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            float2 e;
            if constexpr (MK == 0)
              e = __ffma2_rn(pf2(xs[2 * c], xs[2 * c + 1]), c2, nm2);
            else
              e = __fadd2_rn(pf2(xs[2 * c], xs[2 * c + 1]), nm2);
            const float2 pv = make_float2(fast_exp2(e.x), fast_exp2(e.y));
            ls2 = __fadd2_rn(ls2, pv);
            pp[16 * hh + c] = Elem<T>::pack(pv.x, pv.y);
            if constexpr (DUAL) {
              const float2 w = __fmul2_rn(pv, __fmul2_rn(pf2(ts[2 * c], ts[2 * c + 1]), sc2));
              ms2 = __fadd2_rn(ms2, w);
              wp[16 * hh + c] = Elem<T>::pack(w.x, w.y);
            }
          }
        }
        l_run = l_run * alpha + (ls2.x + ls2.y);
        if constexpr (DUAL) mu_run = mu_run * alpha + (ms2.x + ms2.y);
        // The P / W tiles are single-buffered: the previous tile's output MMAs must have read them.
        if (t > 0 && !prev_pv_seen && !mbar_wait(pv_done + X, (t - 1) & 1, ab, kAbortOFull)) {
          alive = false;
          break;
        }
        if (first && !release_staging()) {  // the previous item's output store has read the buffers
          alive = false;
          break;
        }
        if constexpr (DUAL) {
#pragma unroll
          for (int c = 0; c < 8; ++c) {  // chunk c = key columns 8c .. 8c+7
            const uint32_t off = ((uint32_t)c ^ sw) << 4;
            st_shared_v4(pP + off, pp[4 * c], pp[4 * c + 1], pp[4 * c + 2], pp[4 * c + 3]);
            st_shared_v4(pW + off, wp[4 * c], wp[4 * c + 1], wp[4 * c + 2], wp[4 * c + 3]);
          }
          fence_proxy_async_smem();
        } else {
          tmem_st32(tq + C::COL_P, pp);
          tmem_wait_st();
        }
        tc_fence_before();
        mbar_arrive(p_full + X);
        first = false;
        ++t;
      }
      if (!alive) break;
      if (!epilogue(it, i, m_used, l_run, mu_run, true)) break;
      ++kx;
    }
    (void)kx;
    if (row == 0) tma_store_wait_all();  // shared memory must outlive the stores that read it
  }
  tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0) poison();
  if (warp == 0) {
    if (*abort_flag != 0) {
      // Something gave up: give copies and MMAs that may still be in flight time to land before the TMEM
      // columns go back to the allocator.
      const long long t0 = clock64();
      while (clock64() - t0 < (1ll << 22)) {
      }
    }
    tc_fence_after();
    tmem_dealloc(tmem, C::COLS_ALLOC);
  }
}

static int pair_sm_count() {
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
static int launch_pair64(const jvpfa_fwd_args& a, cudaStream_t stream) {
  using C = FwdPairCfg<DUAL>;
  int* status = tc5_status_device_ptr();
  if (!status) {
    set_last_cuda_error(cudaErrorUnknown, "status word address");
    return JVPFA_ERR_CUDA;
  }
  FwdPairMaps maps;
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
  ok = ok && encode_map4(&maps.o, dt, a.o, a.L, a.H, a.B, nullptr, C::BM);
  if (DUAL)
    ok = ok && encode_map4(&maps.to, dt, a.to, a.L, a.H, a.B, nullptr, C::BM);
  else
    maps.to = maps.o;
  if (!ok) {
    set_last_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled(fwd pair64)");
    return JVPFA_ERR_CUDA;
  }
  auto kern = fwd_tc5_pair64_kernel<T, DUAL, MK>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
  if (e != cudaSuccess) {
    set_last_cuda_error(e, "cudaFuncSetAttribute(fwd_tc5_pair64)");
    return JVPFA_ERR_CUDA;
  }
  const int sms = pair_sm_count();
  if (sms <= 0) {
    set_last_cuda_error(cudaErrorUnknown, "multiprocessor count");
    return JVPFA_ERR_CUDA;
  }
  const long long n_q_tiles = (a.L + C::BM - 1) / C::BM;
  const long long n_items = ((n_q_tiles + 1) / 2) * BH;
  const int grid = (int)(n_items < sms ? n_items : sms);
  kern<<<grid, C::NTHREADS, C::SMEM_BYTES, stream>>>(a, maps, status);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_cuda_error(e, "launch fwd_tc5_pair64");
    return JVPFA_ERR_CUDA;
  }
  return JVPFA_OK;
}

template <typename T>
static int launch_pair64_t(const jvpfa_fwd_args& a, cudaStream_t s) {
  const bool dual = a.tq != nullptr;
  if (a.mask.kind == JVPFA_MASK_BOOL && a.mask_tile_live != nullptr)
    return dual ? launch_pair64<T, true, 3>(a, s) : launch_pair64<T, false, 3>(a, s);
  if (a.mask.kind == JVPFA_MASK_BOOL) return dual ? launch_pair64<T, true, 1>(a, s) : launch_pair64<T, false, 1>(a, s);
  if (a.mask.kind == JVPFA_MASK_BIAS) return dual ? launch_pair64<T, true, 2>(a, s) : launch_pair64<T, false, 2>(a, s);
  return dual ? launch_pair64<T, true, 0>(a, s) : launch_pair64<T, false, 0>(a, s);
}

}  // namespace tc5

int launch_fwd_tc5_pair64(const jvpfa_fwd_args& a, cudaStream_t s) {
  return a.dtype == JVPFA_BF16 ? tc5::launch_pair64_t<__nv_bfloat16>(a, s) : tc5::launch_pair64_t<__half>(a, s);
}

}  // namespace jvpfa
