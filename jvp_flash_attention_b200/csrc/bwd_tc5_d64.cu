// Persistent, pipelined tcgen05 backward for head dimension 64 (bf16 / fp16; none, causal, key
// padding).
//
// Same mathematics and the same two launches as bwd_tc5.cu (own 128 keys -> dK, dV; own 128
// queries -> dQ), organised around what was measured on B200:
//   (1) one thread issues a tcgen05.mma about every 60-100 cycles whatever N <= 128 is, several
//       issuing warps scale almost linearly;
//   (2) a hand-off through an mbarrier costs ~200 cycles (MMA -> commit -> waiter ~300), so the life
//       of one 32-row sub-tile (scores -> elementwise -> second-stage MMAs -> accumulators free again)
//       is ~2200-3300 cycles against ~500 cycles of tensor work: throughput = that latency divided
//       by the number of sub-tiles in flight;
//   (3) a CTA that owns all of TMEM cannot overlap its start-up and wind-down with another CTA.
// Hence:
//  * one CTA per SM stays resident and walks a static, weight-balanced list of work items
//    (own tile, batch*head): barriers and TMEM are set up once, the TMA producer runs ahead across
//    item boundaries, the next item's own tiles are fetched into the other half of a double-buffered
//    staging area while the current item computes, and the previous item's outputs are converted
//    and stored while the next item's first scores are already being formed;
//  * three sub-tiles are in flight: the four score accumulators of a sub-tile take 128 TMEM columns
//    and exist three times.  That leaves 128 columns: dK and dV (own keys), or dQ and the packed
//    rows of Q and tQ as TMEM-resident A operands (own queries).  All other own-side operands are
//    read from the staging area by shared-memory-descriptor MMAs;
//  * the streamed side advances in sub-tiles of 32 rows through a TMA ring;
//  * three warps issue MMAs, each owning fixed accumulator chains (listed at the issuer code); where
//    two accumulators share the A operand and their B tiles are neighbours in shared memory
//    ([Q;tQ], [K;tK], [V;tV]) one N=64 instruction fills both.  An issuer forms the scores of
//    sub-tile g+2 before the second stage of sub-tile g, so it never waits for its own MMAs;
//  * two elementwise warpgroups alternate over the sub-tiles: they turn the accumulators into the
//    16-bit operands (P, A, gtS, gS, written back in place) with packed fp32x2 arithmetic and
//    selects instead of branches.
//
// TMEM map (512 columns):  buffer b at 128*b: S | TS | E | FP (32 each), b = 0..2 ; OUT0 at 384
// (64) ; own keys: OUT1 at 448 (64) ; own queries: packed Q at 448, tQ at 480.
// Sub-tiles are numbered globally over the CTA's items (index g): stage g % STAGES, buffer g % 3,
// elementwise group g & 1.
// Barriers: loop_full/loop_empty[stage]; s_full[b] (one arrival per score issuer) -> elementwise;
// p_full[b] (128 threads) -> second-stage issuers; loop_empty[stage] (one arrival per second-stage
// issuer) also releases buffer b to the score issuers.  Per item: own_staged[h] (TMA, staging half
// h) -> issuers / elementwise; own_free[h] (256 threads) -> producer; own_ready (256 threads, own
// queries only: packed rows are in TMEM) -> issuers; done (second-stage issuers) -> elementwise;
// out_free (256 threads) -> second-stage issuers of the next item.
#include "tc5_common.cuh"

namespace jvpfa {
namespace tc5 {

struct Bwd64Maps {
  CUtensorMap k, v, tk, tv;  // key-side tensors
  CUtensorMap q, go, tq, g;  // query-side tensors (g = cotangent of tO)
  // own side: box 128 rows, streamed side: box 32 rows
};

template <bool OWN_KEYS, bool HAS_GO, bool HAS_GT>
struct Bwd64Cfg {
  static constexpr int D = 64;
  static constexpr int OWN = 128;
  static constexpr int BL = 32;
  static constexpr int NBUF = 3;                                // sub-tiles in flight
  static constexpr int STAGES = (HAS_GO && HAS_GT) ? 5 : 6;     // TMA ring depth (limited by shared memory)
  // warp 0: TMA producer; warps 1, 2 and 13, 14: score issuers (two per sub-tile, even / odd
  // sub-tiles); warp 3: second-stage issuer (dK or dQ); warps 4..11: two elementwise warpgroups;
  // warp 12: second-stage issuer for dV (own keys; idle otherwise)
  static constexpr int NTHREADS = 480;
  static constexpr int N_SCORE_THREADS = 4;
  static constexpr int N_OUT_ISSUERS = OWN_KEYS ? 2 : 1;
  // s_full barriers are indexed by g % 6: sub-tiles that share one have the same accumulator buffer
  // (g % 3) and the same elementwise group (g & 1), so its waiter sees every phase.
  static constexpr int N_SFULL = 6;
  static constexpr int N_KEY_TILES = HAS_GT ? 4 : 2;
  static constexpr int N_QRY_TILES = 1 + (HAS_GO ? 1 : 0) + (HAS_GT ? 2 : 0);
  static constexpr int N_OWN = OWN_KEYS ? N_KEY_TILES : N_QRY_TILES;
  static constexpr int N_LOOP = OWN_KEYS ? N_QRY_TILES : N_KEY_TILES;
  static constexpr int N_OUT_BUF = OWN_KEYS ? 1 : 2;  // own queries: dQ accumulator exists twice
  static constexpr int LOOP_BYTES = BL * D * 2;  // 4 KiB
  static constexpr int OWN_BYTES = OWN * D * 2;  // 16 KiB
  static constexpr int STAGE_BYTES = N_LOOP * LOOP_BYTES;
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  static constexpr int STAGING_HALF = N_OWN * OWN_BYTES;
  static constexpr int STAGING_BYTES = 2 * STAGING_HALF;
  static constexpr int STAT_BYTES = OWN_KEYS ? STAGES * (BL / 2) * 32 : 0;  // two float4 per column pair
  static constexpr int TILE_BYTES = RING_BYTES + STAGING_BYTES;
  // At least 120 KiB so that a second CTA can never share the SM (the CTA allocates all of TMEM).
  static constexpr int SMEM_NEEDED = TILE_BYTES + STAT_BYTES + 512 + 1024;
  static constexpr int SMEM_BYTES = SMEM_NEEDED > 120 * 1024 ? SMEM_NEEDED : 120 * 1024;
  static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
  static constexpr int COL_BUF = 128;  // columns per accumulator buffer
  static constexpr int OFF_S = 0, OFF_TS = 32, OFF_E = 64, OFF_FP = HAS_GT ? 96 : 32;
  static constexpr int COL_OUT0 = NBUF * COL_BUF, COL_OUT1 = COL_OUT0 + 64;  // own queries: second dQ at COL_OUT1
  static constexpr int COLS_ALLOC = 512;
  // Tile slots (staging tiles of the own side, ring tiles of the streamed side, TMEM operand slots).
  // K|tK, V|tV and Q|tQ are neighbours so that one N=64 instruction can take both as its B operand.
  static constexpr int SLOT_K = 0, SLOT_TK = 1, SLOT_V = HAS_GT ? 2 : 1, SLOT_TV = 3;
  static constexpr int SLOT_Q = 0, SLOT_TQ = 1, SLOT_G = 2, SLOT_GO = HAS_GT ? 3 : 1;
};

__device__ __forceinline__ float2 f2(uint32_t a, uint32_t b) { return make_float2(__uint_as_float(a), __uint_as_float(b)); }

// One work item of the persistent loop.
struct BwdItem {
  int bh, b, h, own0, loop_begin, n_sub;
  // MK = 3: the item's words of the tile bitmap (bit t: streamed tile t has a true entry) and how many
  // 32-row sub-tiles one bit stands for; sparse == false: every sub-tile from loop_begin is visited.
  unsigned long long w0, w1;
  int per_bit;
  bool sparse;
};

// Position of the n-th (0-based) set bit of the 128-bit word (w1:w0); the caller guarantees it exists.
__device__ __forceinline__ int nth_set_bit(unsigned long long w0, unsigned long long w1, int n) {
  const uint32_t part[4] = {(uint32_t)w0, (uint32_t)(w0 >> 32), (uint32_t)w1, (uint32_t)(w1 >> 32)};
  int pos = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = __popc(part[i]);
    if (n < c) return pos + (int)__fns(part[i], 0u, n + 1);
    n -= c;
    pos += 32;
  }
  return 127;
}

// First streamed row of the item's s-th visited sub-tile.
template <int BL>
__device__ __forceinline__ int sub_l0(const BwdItem& it, int s) {
  if (!it.sparse) return it.loop_begin + s * BL;
  const int t = nth_set_bit(it.w0, it.w1, s / it.per_bit);
  return (t * it.per_bit + s % it.per_bit) * BL;
}

// MK: 0 = none / causal / key padding (index comparisons); 1 = uint8 mask; 2 = additive bias of the
// element type T.  For 1 and 2 an elementwise thread fetches its own row's share of the sub-tile from
// global memory before it waits for the sub-tile's scores: with own queries 32 consecutive mask
// elements (16-byte loads), with own keys one element of each of the 32 query rows (lanes read
// neighbouring keys).  The key stride must be 1, rows 16-byte aligned and L a multiple of 16.
template <typename T, bool OWN_KEYS, bool HAS_GO, bool HAS_GT, int MK>
__global__ void __launch_bounds__(480, 1)
bwd_tc5_d64_kernel(const jvpfa_bwd_args a, const __grid_constant__ Bwd64Maps maps, int* status) {
  using C = Bwd64Cfg<OWN_KEYS, HAS_GO, HAS_GT>;
  constexpr int D = 64, OWN = C::OWN, BL = C::BL, STAGES = C::STAGES, NBUF = C::NBUF;

  // The own-queries launch that follows an own-keys launch reads nothing this kernel writes, so it is
  // launched with programmatic stream serialization and may take over each SM as soon as this
  // kernel's CTA there has exited (both need a whole SM): the tails of the two launches overlap.
  if constexpr (OWN_KEYS) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const bool dead_on_entry = *(volatile int*)status != 0;  // an earlier bounded wait gave up

  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  unsigned char* smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  unsigned char* sLoop = smem;
  unsigned char* sOwn = smem + C::RING_BYTES;                        // two halves of N_OWN tiles
  float4* sStat = reinterpret_cast<float4*>(smem + C::TILE_BYTES);  // [STAGES][BL/2][2]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::TILE_BYTES + C::STAT_BYTES);
  uint64_t* loop_full = bars;                // [STAGES]
  uint64_t* loop_empty = bars + STAGES;      // [STAGES]
  uint64_t* s_full = bars + 2 * STAGES;      // [N_SFULL]
  uint64_t* p_full = s_full + C::N_SFULL;    // [NBUF]
  uint64_t* own_staged = p_full + NBUF;      // [2]
  uint64_t* own_free = own_staged + 2;       // [2]
  uint64_t* done = own_free + 2;             // [2] (per output buffer)
  uint64_t* out_free = done + 2;             // [2] (per output buffer)
  uint64_t* stat_full = out_free + 2;        // [STAGES] (own keys: row statistics of the stage are in place)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(stat_full + STAGES);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int L = a.L;
  const int BH = a.B * a.H;
  const bool causal = a.mask.kind == JVPFA_MASK_CAUSAL;
  const int n_own_tiles = (L + OWN - 1) / OWN;
  const int n_items = n_own_tiles * BH;
  const int G = (int)gridDim.x, cta = (int)blockIdx.x;

  // Item k of this CTA.  Items are ranked heaviest first (for causal masks the own tile decides the
  // weight) and dealt to the CTAs in serpentine order, which keeps the per-CTA sums balanced.
  auto get_item = [&](int k, BwdItem& it) -> bool {
    const int w = k * G + ((k & 1) ? (G - 1 - cta) : cta);
    if (w >= n_items) return false;
    const int rank = w / BH;
    it.bh = w - rank * BH;
    it.b = it.bh / a.H;
    it.h = it.bh - it.b * a.H;
    int n_valid = L;
    if (a.mask.kind == JVPFA_MASK_KVLEN) {
      const int n = a.mask.kv_len[it.b];
      n_valid = n < 0 ? 0 : (n > L ? L : n);
    }
    if constexpr (OWN_KEYS) {
      it.own0 = rank * OWN;
      it.loop_begin = causal ? (it.own0 / BL) * BL : 0;
      it.n_sub = (L - it.loop_begin + BL - 1) / BL;
      if (it.own0 >= n_valid) it.n_sub = 0;
    } else {
      it.own0 = (n_own_tiles - 1 - rank) * OWN;
      it.loop_begin = 0;
      int n_end = n_valid;
      if (causal) n_end = min(n_end, it.own0 + OWN);
      it.n_sub = (n_end + BL - 1) / BL;
    }
    it.sparse = false;
    it.w0 = it.w1 = 0ull;
    it.per_bit = 1;
    if constexpr (MK == 3) {
      // Bitmaps have the mask's own extents: a broadcast dimension (stride 0) has one entry.
      const long long hm = (a.mask.stride[0] ? (long long)it.b * (a.mask.stride[1] ? a.H : 1) : 0) +
                           (a.mask.stride[1] ? it.h : 0);
      const int n_t128 = (L + 127) / 128;
      const bool rows = a.mask.stride[2] != 0;
      if constexpr (OWN_KEYS) {
        // bit qt of the transposed bitmap's entry [head][own 128-key tile]: four 32-query sub-tiles each
        const int n_words_t = rows ? (n_t128 + 63) / 64 : 1;
        const unsigned long long* w =
            reinterpret_cast<const unsigned long long*>(a.mask_tile_live_t) + (hm * n_t128 + it.own0 / OWN) * n_words_t;
        if (!rows) {  // one mask row for all queries: the own tile is live for all of them or for none
          if (!(__ldg(w) & 1ull)) it.n_sub = 0;
        } else {
          it.w0 = __ldg(w);
          it.w1 = n_words_t > 1 ? __ldg(w + 1) : 0ull;
          it.per_bit = 128 / BL;
          it.sparse = true;
        }
      } else {
        // bit kt of the bitmap's entry [head][own 128-query tile]: 64-key tiles, two 32-key sub-tiles each
        const int n_words = ((L + 63) / 64 + 63) / 64;
        const unsigned long long* w = reinterpret_cast<const unsigned long long*>(a.mask_tile_live) +
                                      (rows ? hm * n_t128 + it.own0 / OWN : hm) * n_words;
        it.w0 = __ldg(w);
        it.w1 = n_words > 1 ? __ldg(w + 1) : 0ull;
        it.per_bit = 64 / BL;
        it.sparse = true;
      }
      if (it.sparse) {
        const int n_bits = __popcll(it.w0) + __popcll(it.w1);
        int n = n_bits * it.per_bit;
        if (n_bits > 0) {  // the highest live tile may reach past L
          const int top = it.w1 ? 127 - __clzll(it.w1) : 63 - __clzll(it.w0);
          const int rows_left = L - top * it.per_bit * BL;
          const int subs_top = min(it.per_bit, (rows_left + BL - 1) / BL);
          n -= it.per_bit - subs_top;
        }
        it.n_sub = n;
      }
    }
    return true;
  };
  const int k_max = (n_items + G - 1) / G;
  // Advances k to the next item that has work; false when the list is exhausted.
  auto next_active = [&](int& k, BwdItem& it) -> bool {
    for (; k < k_max; ++k)
      if (get_item(k, it) && it.n_sub > 0) return true;
    return false;
  };
  auto valid_keys = [&](int b) {
    int n_valid = L;
    if (a.mask.kind == JVPFA_MASK_KVLEN) {
      const int n = a.mask.kv_len[b];
      n_valid = n < 0 ? 0 : (n > L ? L : n);
    }
    return n_valid;
  };

  // NaN into the output rows that this CTA's items own: this launch's results are not to be trusted
  auto poison = [&]() {
    BwdItem it;
    for (int k = 0; k < k_max; ++k) {
      if (!get_item(k, it)) continue;
      const int i = it.own0 + tid;
      if (tid < OWN && i < L) {
        if constexpr (OWN_KEYS) {
          poison_row<T>(a.dk, (size_t)it.bh * L + i, D);
          poison_row<T>(a.dv, (size_t)it.bh * L + i, D);
        } else {
          poison_row<T>(a.dq, (size_t)it.bh * L + i, D);
        }
      }
    }
  };
  if (dead_on_entry) {
    poison();
    // the stream's next kernel must still be ordered after the launch this one overlaps
    if constexpr (!OWN_KEYS) asm volatile("griddepcontrol.wait;" ::: "memory");
    return;
  }

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(loop_full + s, 1);
      mbar_init(stat_full + s, 1);
      mbar_init(loop_empty + s, C::N_OUT_ISSUERS);
    }
    for (int b = 0; b < C::N_SFULL; ++b) mbar_init(s_full + b, 2);  // the two score threads of a sub-tile
    for (int b = 0; b < NBUF; ++b) mbar_init(p_full + b, 128);
    // The score threads take part in own_free (see below).
    for (int h = 0; h < 2; ++h) {
      mbar_init(own_staged + h, 1);
      mbar_init(own_free + h, 256 + C::N_SCORE_THREADS);
      mbar_init(out_free + h, 256);
      mbar_init(done + h, C::N_OUT_ISSUERS);
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

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (+ stats)
    if (lane == 0) {
      prefetch_tmap(&maps.k), prefetch_tmap(&maps.v), prefetch_tmap(&maps.q);
      if constexpr (HAS_GO) prefetch_tmap(&maps.go);
      if constexpr (HAS_GT) prefetch_tmap(&maps.tk), prefetch_tmap(&maps.tv), prefetch_tmap(&maps.tq), prefetch_tmap(&maps.g);
    }
    // Own tiles of active item number j -> staging half j & 1 (free once item j - 2 is complete).
    auto load_own = [&](const BwdItem& it, int j) -> bool {
      const int h = j & 1, use = j >> 1;
      if (use > 0 && !mbar_wait(own_free + h, (use - 1) & 1, ab, kAbortBwdOwn)) return false;
      if (lane == 0) {
        unsigned char* dst = sOwn + h * C::STAGING_HALF;
        mbar_expect_tx(own_staged + h, C::STAGING_HALF);
        if constexpr (OWN_KEYS) {
          tma_load_4d(dst + C::SLOT_K * C::OWN_BYTES, &maps.k, own_staged + h, 0, it.own0, it.h, it.b);
          tma_load_4d(dst + C::SLOT_V * C::OWN_BYTES, &maps.v, own_staged + h, 0, it.own0, it.h, it.b);
          if constexpr (HAS_GT) {
            tma_load_4d(dst + C::SLOT_TK * C::OWN_BYTES, &maps.tk, own_staged + h, 0, it.own0, it.h, it.b);
            tma_load_4d(dst + C::SLOT_TV * C::OWN_BYTES, &maps.tv, own_staged + h, 0, it.own0, it.h, it.b);
          }
        } else {
          tma_load_4d(dst + C::SLOT_Q * C::OWN_BYTES, &maps.q, own_staged + h, 0, it.own0, it.h, it.b);
          if constexpr (HAS_GO) tma_load_4d(dst + C::SLOT_GO * C::OWN_BYTES, &maps.go, own_staged + h, 0, it.own0, it.h, it.b);
          if constexpr (HAS_GT) {
            tma_load_4d(dst + C::SLOT_TQ * C::OWN_BYTES, &maps.tq, own_staged + h, 0, it.own0, it.h, it.b);
            tma_load_4d(dst + C::SLOT_G * C::OWN_BYTES, &maps.g, own_staged + h, 0, it.own0, it.h, it.b);
          }
        }
      }
      return true;
    };
    int gbase = 0, kact = 0, k = 0;
    BwdItem it, nxt;
    bool have = next_active(k, it);
    bool ok = have ? load_own(it, 0) : true;
    while (ok && have) {
      int k2 = k + 1;
      const bool have_next = next_active(k2, nxt);
      bool next_loaded = !have_next;
      const size_t stat_off = (size_t)it.bh * L;
      // Own keys: the row statistics of the streamed queries, one query per lane, negated and stored
      // pairwise for the packed arithmetic.  A global load takes longer than a sub-tile, and this loop
      // has nothing else to wait for, so the loads are issued for CH sub-tiles at a time, one chunk
      // ahead of their use.
      constexpr int CH = 4;
      struct Stat {  // raw values: the arithmetic waits until they are used, not until they are loaded
        float lse, delta, mu, eps, cterm;
      };
      auto load_stats = [&](int s_first, Stat(&r)[CH]) {
#pragma unroll
        for (int j = 0; j < CH; ++j) {
          r[j] = Stat{INFINITY, 0.f, 0.f, 0.f, 0.f};
          if (s_first + j >= it.n_sub) continue;
          const int i = sub_l0<BL>(it, s_first + j) + lane;
          if (i < L) {
            r[j].lse = a.lse[stat_off + i];
            r[j].delta = a.delta[stat_off + i];
            if constexpr (HAS_GT) {
              r[j].mu = a.mu[stat_off + i];
              r[j].eps = a.eps[stat_off + i];
              r[j].cterm = a.cterm[stat_off + i];
            }
          }
        }
      };
      auto put_stats = [&](int st, const Stat& v) {
        float* base = reinterpret_cast<float*>(sStat + (st * (BL / 2) + (lane >> 1)) * 2);
        base[(lane & 1)] = -v.lse;      // float4 A = (-lse0, -lse1, -mu0, -mu1)
        base[2 + (lane & 1)] = -v.mu;
        base[4 + (lane & 1)] = -v.eps;  // float4 B = (-eps0, -eps1, -sub0, -sub1)
        base[6 + (lane & 1)] = -(v.delta + v.cterm + v.eps * v.mu);
        __syncwarp();
        if (lane == 0) mbar_arrive(stat_full + st);
      };
      Stat cur[CH], ahead[CH];
      if constexpr (OWN_KEYS) load_stats(0, cur);
      for (int s0 = 0; ok && s0 < it.n_sub; s0 += CH) {
        if constexpr (OWN_KEYS) load_stats(s0 + CH, ahead);
#pragma unroll
        for (int j = 0; j < CH; ++j) {
          const int s = s0 + j;
          if (!ok || s >= it.n_sub) continue;
          // The next item's own tiles go out once the ring is full: by then its staging half is free.
          if (s == STAGES && !next_loaded) {
            ok = load_own(nxt, kact + 1);
            next_loaded = true;
            if (!ok) continue;
          }
          const int g = gbase + s;
          const int st = g % STAGES;
          const uint32_t ph = (g / STAGES) & 1;
          if (!mbar_wait(loop_empty + st, ph ^ 1, ab, kAbortBwdLoopEmpty)) {
            ok = false;
            continue;
          }
          const int l0 = sub_l0<BL>(it, s);
          if (lane == 0) {
            unsigned char* base = sLoop + st * C::STAGE_BYTES;
            mbar_expect_tx(loop_full + st, C::STAGE_BYTES);
            if constexpr (OWN_KEYS) {
              tma_load_4d(base + C::SLOT_Q * C::LOOP_BYTES, &maps.q, loop_full + st, 0, l0, it.h, it.b);
              if constexpr (HAS_GO) tma_load_4d(base + C::SLOT_GO * C::LOOP_BYTES, &maps.go, loop_full + st, 0, l0, it.h, it.b);
              if constexpr (HAS_GT) {
                tma_load_4d(base + C::SLOT_TQ * C::LOOP_BYTES, &maps.tq, loop_full + st, 0, l0, it.h, it.b);
                tma_load_4d(base + C::SLOT_G * C::LOOP_BYTES, &maps.g, loop_full + st, 0, l0, it.h, it.b);
              }
            } else {
              tma_load_4d(base + C::SLOT_K * C::LOOP_BYTES, &maps.k, loop_full + st, 0, l0, it.h, it.b);
              tma_load_4d(base + C::SLOT_V * C::LOOP_BYTES, &maps.v, loop_full + st, 0, l0, it.h, it.b);
              if constexpr (HAS_GT) {
                tma_load_4d(base + C::SLOT_TK * C::LOOP_BYTES, &maps.tk, loop_full + st, 0, l0, it.h, it.b);
                tma_load_4d(base + C::SLOT_TV * C::LOOP_BYTES, &maps.tv, loop_full + st, 0, l0, it.h, it.b);
              }
            }
          }
          if constexpr (OWN_KEYS) put_stats(st, cur[j]);
        }
        if constexpr (OWN_KEYS) {
#pragma unroll
          for (int j = 0; j < CH; ++j) cur[j] = ahead[j];
        }
      }
      if (ok && !next_loaded) ok = load_own(nxt, kact + 1);
      gbase += it.n_sub;
      ++kact;
      it = nxt;
      k = k2;
      have = have_next;
    }
  } else if (warp <= 3 || warp >= 12) {
    // ------------------------------------------------------------------ MMA issuers
    // Each of these warps works with one thread.  Such a thread pays ~75 cycles per MMA and a few
    // hundred cycles of waits and bookkeeping per sub-tile, and the time a sub-tile's scores take to
    // issue is part of the latency that the three buffers in flight have to cover.  So the scores of
    // the even sub-tiles belong to warps 1 and 13, those of the odd sub-tiles to warps 2 and 14:
    //   own keys   : warps 1, 2: [S|TS] = K [Q;tQ]^T, TS += tK Q^T ; warps 13, 14: E = V G^T, FP = tV G^T (+ V gO^T)
    //   own queries: warps 1, 2: [S|TS] = Q [K;tK]^T, TS += tQ K^T ; warps 13, 14: [E|FP] = G [V;tV]^T (+ FP += gO V^T)
    // and the output accumulators, which run through all sub-tiles of an item, have a thread each:
    //   warp 3 : dK += gS^T Q + gtS^T tQ   or   dQ += gS K + gtS tK
    //   warp 12: dV += A^T G (+ P^T gO)    (own keys only)
    // Stage / buffer indices, parities, barrier addresses and descriptor words live in registers
    // and advance by additions.
    constexpr uint32_t idesc_sc = make_idesc(Fmt<T>::kIdesc, OWN, BL, 0, 0);       // 128 x 32 scores
    constexpr uint32_t idesc_sc2 = make_idesc(Fmt<T>::kIdesc, OWN, 2 * BL, 0, 0);  // 128 x 64: two neighbours
    constexpr uint32_t idesc_out = make_idesc(Fmt<T>::kIdesc, OWN, D, 0, 1);       // 128 x 64 outputs
    constexpr uint32_t STAGE16 = C::STAGE_BYTES >> 4, LOOP16 = C::LOOP_BYTES >> 4, OWN16 = C::OWN_BYTES >> 4;
    // A position in the sequence of sub-tiles: ring stage and accumulator buffer with their parities.
    struct Cursor {
      uint32_t st_bar, st_tile, st_par, buf_bar, buf_col, buf_par, sf_bar;
      __device__ __forceinline__ explicit Cursor(uint32_t g)  // g < min(STAGES, NBUF)
          : st_bar(8 * g), st_tile(g * STAGE16), st_par(0), buf_bar(8 * g), buf_col(g * C::COL_BUF), buf_par(0),
            sf_bar(8 * g) {}
      __device__ __forceinline__ void advance(uint32_t n) {  // n = 1 or 2
        st_bar += 8 * n, st_tile += n * STAGE16;
        if (st_bar >= 8 * STAGES) st_bar -= 8 * STAGES, st_tile -= STAGES * STAGE16, st_par ^= 1;
        buf_bar += 8 * n, buf_col += n * C::COL_BUF;
        if (buf_bar >= 8 * NBUF) buf_bar -= 8 * NBUF, buf_col -= NBUF * C::COL_BUF, buf_par ^= 1;
        sf_bar += 8 * n;
        if (sf_bar >= 8 * C::N_SFULL) sf_bar -= 8 * C::N_SFULL;
      }
    };
    const uint32_t bar_loop_full = smem_u32(loop_full), bar_loop_empty = smem_u32(loop_empty);
    const uint32_t bar_s_full = smem_u32(s_full), bar_p_full = smem_u32(p_full);
    const uint32_t ring_lo = kDescLo | (smem_u32(sLoop) >> 4);

    if (lane == 0 && (warp == 1 || warp == 2 || warp >= 13)) {
      // ---------------- scores of the sub-tiles g = r, r + 2, r + 4, ...
      const bool part_b = warp >= 13;  // which accumulators
      const uint32_t r = part_b ? warp - 13 : warp - 1;
      Cursor cs(r);      // the next sub-tile of this thread
      Cursor cf(1 - r);  // the sub-tile NBUF before the first one (>= NBUF) of this thread: 4 - 3 or 3 - 3
      int g = (int)r;
      uint32_t own_lo = 0;  // descriptor word of the current item's staging half
      // acc (+)= own tile `slot` (A: packed rows in TMEM where they exist, else the staging tile) x
      // streamed tile(s)^T (B, K-major; wide: the tile and its neighbour, 64 rows)
      auto score = [&](uint32_t d, auto slot_c, uint32_t b_lo, auto first_c, auto wide_c) {
        constexpr int slot = decltype(slot_c)::value;
        constexpr bool first = decltype(first_c)::value != 0, wide = decltype(wide_c)::value != 0;
        constexpr uint32_t id = wide ? idesc_sc2 : idesc_sc;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          if (first && ks == 0)
            umma_ss_lo<false>(d, own_lo + slot * OWN16 + ks * 2, b_lo + ks * 2, id);
          else
            umma_ss_lo<true>(d, own_lo + slot * OWN16 + ks * 2, b_lo + ks * 2, id);
        }
      };
      using I0 = IntC<0>;
      using I1 = IntC<1>;
      int gbase = 0, kact = 0;
      bool ok = true;
      BwdItem it;
      for (int k = 0; ok && k < k_max; ++k) {
        if (!get_item(k, it)) continue;
        if (it.n_sub == 0) continue;
        const int g_end = gbase + it.n_sub;
        // This item's own operands: its staging half.  Waited for even when none of the item's sub-tiles
        // is this thread's: a parity wait is only safe for a thread that sees every phase of the barrier.
        ok = mbar_wait(own_staged + (kact & 1), (kact >> 1) & 1, ab, kAbortBwdOwn);
        if (!ok) break;
        tc_fence_after();
        own_lo = kDescLo | (smem_u32(sOwn + (kact & 1) * C::STAGING_HALF) >> 4);
#pragma unroll 1
        for (; g < g_end; g += 2) {
          // The buffer may be overwritten once every second-stage chain of sub-tile g - NBUF has read
          // it: that is what loop_empty[its stage] records (one arrival per second-stage issuer).
          if (g >= NBUF) {
            if (!mbar_wait_u32(bar_loop_empty + cf.st_bar, cf.st_par, ab, kAbortAux)) {
              ok = false;
              break;
            }
            cf.advance(2);
          }
          if (!mbar_wait_u32(bar_loop_full + cs.st_bar, cs.st_par, ab, kAbortBwdLoopFull)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t lp = ring_lo + cs.st_tile;  // tile slot 0 of the stage
          const uint32_t acc = tmem + cs.buf_col;
          if (!part_b) {
            if constexpr (OWN_KEYS) {
              if constexpr (HAS_GT) {
                score(acc + C::OFF_S, IntC<C::SLOT_K>{}, lp + C::SLOT_Q * LOOP16, I1{}, I1{});    // [S|TS] = K [Q;tQ]^T
                score(acc + C::OFF_TS, IntC<C::SLOT_TK>{}, lp + C::SLOT_Q * LOOP16, I0{}, I0{});  // TS += tK Q^T
              } else {
                score(acc + C::OFF_S, IntC<C::SLOT_K>{}, lp + C::SLOT_Q * LOOP16, I1{}, I0{});    // S = K Q^T
              }
            } else {
              if constexpr (HAS_GT) {
                score(acc + C::OFF_S, IntC<C::SLOT_Q>{}, lp + C::SLOT_K * LOOP16, I1{}, I1{});    // [S|TS] = Q [K;tK]^T
                score(acc + C::OFF_TS, IntC<C::SLOT_TQ>{}, lp + C::SLOT_K * LOOP16, I0{}, I0{});  // TS += tQ K^T
              } else {
                score(acc + C::OFF_S, IntC<C::SLOT_Q>{}, lp + C::SLOT_K * LOOP16, I1{}, I0{});    // S = Q K^T
              }
            }
          } else {
            if constexpr (OWN_KEYS) {
              if constexpr (HAS_GT) {
                score(acc + C::OFF_E, IntC<C::SLOT_V>{}, lp + C::SLOT_G * LOOP16, I1{}, I0{});    // E = V G^T
                score(acc + C::OFF_FP, IntC<C::SLOT_TV>{}, lp + C::SLOT_G * LOOP16, I1{}, I0{});  // FP = tV G^T
                if constexpr (HAS_GO) score(acc + C::OFF_FP, IntC<C::SLOT_V>{}, lp + C::SLOT_GO * LOOP16, I0{}, I0{});
              } else {
                score(acc + C::OFF_FP, IntC<C::SLOT_V>{}, lp + C::SLOT_GO * LOOP16, I1{}, I0{});  // FP = V gO^T
              }
            } else {
              if constexpr (HAS_GT) {
                score(acc + C::OFF_E, IntC<C::SLOT_G>{}, lp + C::SLOT_V * LOOP16, I1{}, I1{});    // [E|FP] = G [V;tV]^T
                if constexpr (HAS_GO) score(acc + C::OFF_FP, IntC<C::SLOT_GO>{}, lp + C::SLOT_V * LOOP16, I0{}, I0{});
              } else {
                score(acc + C::OFF_FP, IntC<C::SLOT_GO>{}, lp + C::SLOT_V * LOOP16, I1{}, I0{});  // FP = gO V^T
              }
            }
          }
          tc_commit_u32(bar_s_full + cs.sf_bar);
          cs.advance(2);
        }
        if (!ok) break;
        // "This thread is through with the item": the staging half is not refilled before, so its
        // barrier cannot run more than one phase ahead of this thread.
        mbar_arrive(own_free + (kact & 1));
        gbase = g_end;
        ++kact;
      }
    } else if (lane == 0 && (warp == 3 || (OWN_KEYS && warp == 12))) {
      // ---------------- second stage: one output accumulator through all sub-tiles
      const bool second = warp == 12;  // dV
      Cursor co(0);
      int kact = 0, g = 0;
      bool ok = true;
      BwdItem it;
      // out (+)= packed operand (A, TMEM, 16 columns per 16 streamed rows) x streamed tile (B, MN-major)
      auto outer = [&](uint32_t out_col, uint32_t a_col, uint32_t b_lo, uint32_t accumulate) {
        umma_ts_lo_dyn(tmem + out_col, a_col, b_lo, idesc_out, accumulate);
        umma_ts_lo<true>(tmem + out_col, a_col + 8, b_lo + (2048 >> 4), idesc_out);
      };
      for (int k = 0; ok && k < k_max; ++k) {
        if (!get_item(k, it)) continue;
        if (it.n_sub == 0) continue;
#pragma unroll 1
        for (int s = 0; s < it.n_sub; ++s, ++g) {
          if (!mbar_wait_u32(bar_p_full + co.buf_bar, co.buf_par, ab, kAbortBwdPFull)) {
            ok = false;
            break;
          }
          // The first sub-tile overwrites the output accumulators: the epilogue of the item that used
          // them last must have read them.
          if (s == 0 && kact >= C::N_OUT_BUF &&
              !mbar_wait(out_free + kact % C::N_OUT_BUF, (kact / C::N_OUT_BUF - 1) & 1, ab, kAbortBwdDone)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t lp = ring_lo + co.st_tile;
          const uint32_t opnd = tmem + co.buf_col;
          const uint32_t acc = s > 0;
          if constexpr (OWN_KEYS) {
            if (!second) {
              outer(C::COL_OUT0, opnd + C::OFF_FP, lp + C::SLOT_Q * LOOP16, acc);                        // dK += gS^T Q
              if constexpr (HAS_GT) outer(C::COL_OUT0, opnd + C::OFF_E, lp + C::SLOT_TQ * LOOP16, 1);   // dK += gtS^T tQ
            } else if constexpr (HAS_GT) {
              outer(C::COL_OUT1, opnd + C::OFF_TS, lp + C::SLOT_G * LOOP16, acc);                        // dV += A^T G
              if constexpr (HAS_GO) outer(C::COL_OUT1, opnd + C::OFF_S, lp + C::SLOT_GO * LOOP16, 1);   // dV += P^T gO
            } else {
              outer(C::COL_OUT1, opnd + C::OFF_S, lp + C::SLOT_GO * LOOP16, acc);                        // dV += P^T gO
            }
          } else {
            const uint32_t oc = C::COL_OUT0 + 64 * (kact & 1);
            outer(oc, opnd + C::OFF_FP, lp + C::SLOT_K * LOOP16, acc);                                   // dQ += gS K
            if constexpr (HAS_GT) outer(oc, opnd + C::OFF_E, lp + C::SLOT_TK * LOOP16, 1);              // dQ += gtS tK
          }
          tc_commit_u32(bar_loop_empty + co.st_bar);
          co.advance(1);
        }
        if (ok) tc_commit(done + kact % C::N_OUT_BUF);
        ++kact;
      }
    }
  } else {
    // ------------------------------------------------------------------ elementwise warpgroups
    const int wg = (warp - 4) >> 2;  // 0 / 1: parity of the sub-tiles this group works on
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t tbase = tmem + lane_off;
    const float2 c2 = make_float2(a.sm_scale * kLog2e, a.sm_scale * kLog2e);
    const float2 sc2 = make_float2(a.sm_scale, a.sm_scale);
    bool alive = true;
    int gbase = 0, kact = 0;
    BwdItem it;

    // group 0 stores columns [0,32) of every output, group 1 columns [32,64)
    auto store_half = [&](void* gptr, int bh, int own_idx, const uint32_t (&r)[32], float mul) {
      if (own_idx >= L) return;
      T* gp = reinterpret_cast<T*>(gptr) + ((size_t)bh * L + own_idx) * D + 32 * wg;
      uint32_t pk[16];
#pragma unroll
      for (int x = 0; x < 16; ++x)
        pk[x] = Elem<T>::pack(__uint_as_float(r[2 * x]) * mul, __uint_as_float(r[2 * x + 1]) * mul);
#pragma unroll
      for (int x = 0; x < 4; ++x)
        reinterpret_cast<uint4*>(gp)[x] = make_uint4(pk[4 * x], pk[4 * x + 1], pk[4 * x + 2], pk[4 * x + 3]);
    };

    // Item epilogue: read this group's half of the output accumulators, release them, store.
    int pend_kact = -1, pend_bh = 0, pend_own_idx = 0;
    auto epilogue = [&]() -> bool {
      const int pk = pend_kact;
      pend_kact = -1;
      // (done and out_free exist per output buffer: with two buffers an item can complete without one
      // of the elementwise groups, and a parity wait must not fall two phases behind)
      if (!mbar_wait(done + pk % C::N_OUT_BUF, (pk / C::N_OUT_BUF) & 1, ab, kAbortBwdDone)) {
        alive = false;
        return false;
      }
      tc_fence_after();
      uint32_t r0[32];
      uint32_t r1[OWN_KEYS ? 32 : 1];
      tmem_ld32(tbase + C::COL_OUT0 + (OWN_KEYS ? 0 : 64 * (pk & 1)) + 32 * wg, r0);
      if constexpr (OWN_KEYS) tmem_ld32(tbase + C::COL_OUT1 + 32 * wg, r1);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(out_free + pk % C::N_OUT_BUF);
      mbar_arrive(own_free + (pk & 1));  // every MMA of the item is complete: its staging half is free
      if constexpr (OWN_KEYS) {
        store_half(a.dk, pend_bh, pend_own_idx, r0, a.sm_scale);
        store_half(a.dv, pend_bh, pend_own_idx, r1, 1.f);
      } else {
        store_half(a.dq, pend_bh, pend_own_idx, r0, a.sm_scale);
      }
      return true;
    };
    for (int k = 0; alive && k < k_max; ++k) {
      if (!get_item(k, it)) continue;
      const int own_idx = it.own0 + row;
      if (it.n_sub == 0) {
        // nothing attends these rows (all keys of the tile are padding): the gradients are zero
        uint32_t z[32];
#pragma unroll
        for (int x = 0; x < 32; ++x) z[x] = 0u;
        if constexpr (OWN_KEYS) {
          store_half(a.dk, it.bh, own_idx, z, 0.f);
          store_half(a.dv, it.bh, own_idx, z, 0.f);
        } else {
          store_half(a.dq, it.bh, own_idx, z, 0.f);
        }
        continue;
      }
      const int n_valid = valid_keys(it.b);
      const size_t stat_off = (size_t)it.bh * L;
      // MK != 0: start of this head's mask / bias and its row pitch, in bytes
      constexpr bool BOOLM = MK == 1 || MK == 3;
      constexpr int MESZ = BOOLM ? 1 : 2;
      const unsigned char* mbase = nullptr;
      long long mpitch = 0;
      if constexpr (MK != 0) {
        mbase = reinterpret_cast<const unsigned char*>(a.mask.ptr) +
                ((long long)it.b * a.mask.stride[0] + (long long)it.h * a.mask.stride[1]) * MESZ;
        mpitch = a.mask.stride[2] * MESZ;
      }

      float r_nlse = -INFINITY, r_nmu = 0.f, r_neps = 0.f, r_nsub = 0.f;
      if constexpr (!OWN_KEYS) {
        // row statistics, negated
        if (own_idx < L) {
          r_nlse = -a.lse[stat_off + own_idx];
          float sub = a.delta[stat_off + own_idx];
          if constexpr (HAS_GT) {
            const float mu = a.mu[stat_off + own_idx], eps = a.eps[stat_off + own_idx];
            r_nmu = -mu;
            r_neps = -eps;
            sub += a.cterm[stat_off + own_idx] + eps * mu;
          }
          r_nsub = -sub;
        }
      }

      // sub-tiles whose global index has this group's parity
      for (int s = ((wg - gbase) & 1); s < it.n_sub; s += 2) {
        const int g = gbase + s;
        const int st = g % STAGES, buf = g % NBUF;
        const uint32_t tbuf = tbase + buf * C::COL_BUF;
        const int l0 = sub_l0<BL>(it, s);
        // MK != 0: the thread's 32 mask / bias elements of this sub-tile, requested before the waits.
        // Indices are clamped into the tensor; what lies outside is switched off by col_lo / col_hi below.
        constexpr int NRAW = MK == 0 ? 1 : (OWN_KEYS ? 32 : 8 * MESZ);
        uint32_t raw[NRAW];
        if constexpr (MK != 0) {
          if constexpr (OWN_KEYS) {
            const unsigned char* p = mbase + (long long)min(own_idx, L - 1) * MESZ;
#pragma unroll
            for (int col = 0; col < 32; ++col) {
              const unsigned char* e = p + (long long)min(l0 + col, L - 1) * mpitch;
              raw[col] = BOOLM ? ldg_nc_u8(e) : ldg_nc_u16(e);
            }
          } else {
            const unsigned char* p = mbase + (long long)min(own_idx, L - 1) * mpitch + (size_t)l0 * MESZ;
#pragma unroll
            for (int j = 0; j < 2 * MESZ; ++j) {
              uint4 r = make_uint4(0u, 0u, 0u, 0u);
              if (l0 + (j + 1) * (16 / MESZ) <= L) r = ldg_nc_v4(p + 16 * j);
              raw[4 * j] = r.x, raw[4 * j + 1] = r.y, raw[4 * j + 2] = r.z, raw[4 * j + 3] = r.w;
            }
          }
        }
        if constexpr (OWN_KEYS) {
          if (!mbar_wait(stat_full + st, (g / STAGES) & 1, ab, kAbortBwdLoopFull)) {
            alive = false;
            break;
          }
        }
        if (!mbar_wait(s_full + g % C::N_SFULL, (g / C::N_SFULL) & 1, ab, kAbortBwdSFull)) {
          alive = false;
          break;
        }
        tc_fence_after();
        // Masking by index comparison; columns outside [col_lo, col_hi) get p = 0.
        //   own keys   : (key j = own_idx, query i = l0 + col) is dead if j >= n_valid, or causal and j > i
        //   own queries: (query i = own_idx, key j = l0 + col) is dead if j >= n_valid, or causal and j > i
        int col_lo = 0, col_hi = BL;
        if constexpr (OWN_KEYS) {
          if (own_idx >= n_valid) col_hi = 0;
          if (causal) col_lo = own_idx - l0;  // i >= j  <=>  col >= j - l0
        } else {
          col_hi = min(BL, n_valid - l0);
          if (causal) col_hi = min(col_hi, own_idx - l0 + 1);  // j <= i
        }
        // MK = 1: bit col of live = column col may attend (mask and index range together);
        // MK = 2: mb[x] = the bias of columns 2x, 2x+1 as a packed pair
        uint32_t live = 0xffffffffu;
        uint32_t mb[MK == 2 ? 16 : 1];
        if constexpr (BOOLM) {
          live = 0u;
          if constexpr (OWN_KEYS) {
#pragma unroll
            for (int col = 0; col < 32; ++col) live |= (raw[col] != 0u ? 1u : 0u) << col;
          } else {
#pragma unroll
            for (int w = 0; w < 8; ++w)  // bytes -> 0/1 -> four bits
              live |= (((__vcmpne4(raw[w], 0u) & 0x01010101u) * 0x01020408u) >> 24) << (4 * w);
          }
          const int lo = max(col_lo, 0), hi = min(col_hi, BL);
          live &= hi > lo ? ((hi - lo >= 32 ? 0xffffffffu : ((1u << (hi - lo)) - 1u)) << lo) : 0u;
        }
        if constexpr (MK == 2) {
#pragma unroll
          for (int x = 0; x < 16; ++x) mb[x] = OWN_KEYS ? (raw[2 * x] | (raw[2 * x + 1] << 16)) : raw[x];
        }
        const float4* stat = sStat + st * (BL / 2) * 2;
        // Two halves of 16 columns, as a real loop: the body exists once, which keeps the instruction
        // footprint of the eight elementwise warps small next to the single-thread MMA issuers.
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t sv[16], fp[16], ts[16], ev[16];
          tmem_ld16(tbuf + C::OFF_S + 16 * c, sv);
          tmem_ld16(tbuf + C::OFF_FP + 16 * c, fp);
          if constexpr (HAS_GT) {
            tmem_ld16(tbuf + C::OFF_TS + 16 * c, ts);
            tmem_ld16(tbuf + C::OFF_E + 16 * c, ev);
          }
          tmem_wait_ld();
          const int lo_c = col_lo - 16 * c, hi_c = col_hi - 16 * c;  // live columns of this half: [lo_c, hi_c)
          const uint32_t live_c = live >> (16 * c);
          uint32_t pk_gs[8], pk_gt[8], pk_av[8], pk_p[8];
#pragma unroll
          for (int x = 0; x < 8; ++x) {
            const int col = 2 * x;  // even column of the pair, within the half
            float2 nl, nmu, neps, nsub;
            if constexpr (OWN_KEYS) {
              const float4 sa = stat[(8 * c + x) * 2], sb = stat[(8 * c + x) * 2 + 1];
              nl = make_float2(sa.x, sa.y), nmu = make_float2(sa.z, sa.w);
              neps = make_float2(sb.x, sb.y), nsub = make_float2(sb.z, sb.w);
            } else {
              nl = make_float2(r_nlse, r_nlse), nmu = make_float2(r_nmu, r_nmu);
              neps = make_float2(r_neps, r_neps), nsub = make_float2(r_nsub, r_nsub);
            }
            float2 xs = __ffma2_rn(f2(sv[2 * x], sv[2 * x + 1]), c2, nl);
            if constexpr (MK == 2)  // scores are in log2 units: + bias * log2(e)
              xs = __ffma2_rn(unpack2<T>(c ? mb[8 + x] : mb[x]), make_float2(kLog2e, kLog2e), xs);
            float2 p;
            if constexpr (BOOLM) {
              p.x = (live_c & (1u << col)) ? fast_exp2(xs.x) : 0.f;
              p.y = (live_c & (2u << col)) ? fast_exp2(xs.y) : 0.f;
            } else {
              p.x = (col >= lo_c && col < hi_c) ? fast_exp2(xs.x) : 0.f;
              p.y = (col + 1 >= lo_c && col + 1 < hi_c) ? fast_exp2(xs.y) : 0.f;
            }
            if constexpr (HAS_GT) {
              const float2 tm = __ffma2_rn(f2(ts[2 * x], ts[2 * x + 1]), sc2, nmu);
              const float2 eb = __fadd2_rn(f2(ev[2 * x], ev[2 * x + 1]), neps);
              const float2 av = __fmul2_rn(p, tm);
              const float2 gt = __fmul2_rn(p, eb);
              const float2 u = __fadd2_rn(f2(fp[2 * x], fp[2 * x + 1]), nsub);
              const float2 gs = __fmul2_rn(p, __ffma2_rn(eb, tm, u));
              pk_gs[x] = Elem<T>::pack(gs.x, gs.y);
              pk_gt[x] = Elem<T>::pack(gt.x, gt.y);
              pk_av[x] = Elem<T>::pack(av.x, av.y);
            } else {
              const float2 u = __fadd2_rn(f2(fp[2 * x], fp[2 * x + 1]), nsub);
              const float2 gs = __fmul2_rn(p, u);
              pk_gs[x] = Elem<T>::pack(gs.x, gs.y);
            }
            if constexpr (OWN_KEYS && HAS_GO) pk_p[x] = Elem<T>::pack(p.x, p.y);
          }
          tmem_st8(tbuf + C::OFF_FP + 8 * c, pk_gs);
          if constexpr (HAS_GT) {
            tmem_st8(tbuf + C::OFF_E + 8 * c, pk_gt);
            if constexpr (OWN_KEYS) tmem_st8(tbuf + C::OFF_TS + 8 * c, pk_av);
          }
          if constexpr (OWN_KEYS && HAS_GO) tmem_st8(tbuf + C::OFF_S + 8 * c, pk_p);
        }
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(p_full + buf);
        if (pend_kact >= 0 && !epilogue()) break;
      }
      if (!alive) break;
      // The item's epilogue is deferred until this group has worked on its first sub-tile of the next
      // item: the wait for the item's last MMAs is then covered by useful work.
      if (pend_kact >= 0 && !epilogue()) break;
      pend_kact = kact, pend_bh = it.bh, pend_own_idx = own_idx;
      gbase += it.n_sub;
      ++kact;
    }
    if (alive && pend_kact >= 0) epilogue();
  }

  // The own-queries launch may have started while the own-keys launch before it was still running (programmatic
  // stream serialization).  Whatever follows on the stream is ordered after THIS grid only, so this grid must not
  // complete before that one has: wait for it here, after the work, where the tails of the two launches still overlap.
  if constexpr (!OWN_KEYS) asm volatile("griddepcontrol.wait;" ::: "memory");
  tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0) poison();
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

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
static int sm_count_of_current_device() {
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

template <typename T, bool OWN_KEYS, bool HAS_GO, bool HAS_GT, int MK>
static int launch_half64(const jvpfa_bwd_args& a, cudaStream_t stream, int* status, bool overlap_previous) {
  using C = Bwd64Cfg<OWN_KEYS, HAS_GO, HAS_GT>;
  Bwd64Maps m;
  const long long BH = (long long)a.B * a.H;
  const CUtensorMapDataType dt = Fmt<T>::kTma;
  const int key_rows = OWN_KEYS ? C::OWN : C::BL;
  const int qry_rows = OWN_KEYS ? C::BL : C::OWN;
  // (64, L, H, B) maps; q, k, v and their tangents may be strided views (in_stride), the cotangents are row-major
  const int64_t* st = a.in_stride;
  bool ok = encode_map4(&m.k, dt, a.k, a.L, a.H, a.B, st, key_rows) && encode_map4(&m.v, dt, a.v, a.L, a.H, a.B, st, key_rows) &&
            encode_map4(&m.q, dt, a.q, a.L, a.H, a.B, st, qry_rows);
  m.tk = m.tv = m.k;
  m.go = m.tq = m.g = m.q;
  if (HAS_GO) ok = ok && encode_map4(&m.go, dt, a.go, a.L, a.H, a.B, nullptr, qry_rows);
  if (HAS_GT)
    ok = ok && encode_map4(&m.tk, dt, a.tk, a.L, a.H, a.B, st, key_rows) && encode_map4(&m.tv, dt, a.tv, a.L, a.H, a.B, st, key_rows) &&
         encode_map4(&m.tq, dt, a.tq, a.L, a.H, a.B, st, qry_rows) && encode_map4(&m.g, dt, a.gto, a.L, a.H, a.B, nullptr, qry_rows);
  if (!ok) {
    set_last_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled(bwd d64)");
    return JVPFA_ERR_CUDA;
  }
  const int sms = sm_count_of_current_device();
  if (sms <= 0) {
    set_last_cuda_error(cudaErrorUnknown, "multiprocessor count");
    return JVPFA_ERR_CUDA;
  }
  auto kern = bwd_tc5_d64_kernel<T, OWN_KEYS, HAS_GO, HAS_GT, MK>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
  if (e != cudaSuccess) {
    set_last_cuda_error(e, "cudaFuncSetAttribute(bwd_tc5_d64)");
    return JVPFA_ERR_CUDA;
  }
  const long long n_items = (long long)((a.L + C::OWN - 1) / C::OWN) * BH;
  const int grid = (int)(n_items < sms ? n_items : sms);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid), cfg.blockDim = dim3(C::NTHREADS);
  cfg.dynamicSmemBytes = C::SMEM_BYTES, cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = overlap_previous ? 1 : 0;
  e = cudaLaunchKernelEx(&cfg, kern, a, m, status);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_cuda_error(e, "launch bwd_tc5_d64");
    return JVPFA_ERR_CUDA;
  }
  return JVPFA_OK;
}

template <typename T, bool HAS_GO, bool HAS_GT, int MK>
static int launch_both64(const jvpfa_bwd_args& a, cudaStream_t s) {
  int* status = tc5_status_device_ptr();
  if (!status) {
    set_last_cuda_error(cudaErrorUnknown, "status word address");
    return JVPFA_ERR_CUDA;
  }
  int rc = JVPFA_OK;
  rc = launch_half64<T, true, HAS_GO, HAS_GT, MK>(a, s, status, false);
  if (rc) return rc;
  rc = launch_half64<T, false, HAS_GO, HAS_GT, MK>(a, s, status, true);
  return rc;
}

template <typename T, int MK>
static int launch_mk64(const jvpfa_bwd_args& a, cudaStream_t s) {
  const bool go = a.go != nullptr, gt = a.gto != nullptr;
  if (go && gt) return launch_both64<T, true, true, MK>(a, s);
  if (gt) return launch_both64<T, false, true, MK>(a, s);
  return launch_both64<T, true, false, MK>(a, s);
}

template <typename T>
static int launch_t64(const jvpfa_bwd_args& a, cudaStream_t s) {
  if (a.mask.kind == JVPFA_MASK_BOOL && a.mask_tile_live && a.mask_tile_live_t && a.L <= 8192) return launch_mk64<T, 3>(a, s);
  if (a.mask.kind == JVPFA_MASK_BOOL) return launch_mk64<T, 1>(a, s);
  if (a.mask.kind == JVPFA_MASK_BIAS) return launch_mk64<T, 2>(a, s);
  return launch_mk64<T, 0>(a, s);
}

}  // namespace tc5

int launch_bwd_tc5_d64(const jvpfa_bwd_args& a, cudaStream_t s) {
  return a.dtype == JVPFA_BF16 ? tc5::launch_t64<__nv_bfloat16>(a, s) : tc5::launch_t64<__half>(a, s);
}

}  // namespace jvpfa
