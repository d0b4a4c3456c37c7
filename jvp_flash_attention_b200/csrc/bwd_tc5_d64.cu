// Persistent, pipelined tcgen05 backward for head dimension 64 (bf16 / fp16; none, causal, key
// padding).
//
// Same mathematics and the same two launches as bwd_tc5.cu (own 128 keys -> dK, dV; own 128
// queries -> dQ), organised around what was measured on B200:
//   (1) one thread issues a tcgen05.mma about every 58-70 cycles whatever N <= 64 is, several
//       issuing warps scale almost linearly;
//   (2) with A operands read from shared memory, N <= 64 instructions are bound by the shared
//       memory port, with A in TMEM they are not;
//   (3) a hand-off through an mbarrier costs ~200 cycles (MMA -> commit -> waiter ~300);
//   (4) a CTA that owns all of TMEM cannot overlap its start-up (~7000 cycles) and wind-down (~5000)
//       with another CTA.
// Hence:
//  * one CTA per SM stays resident and walks a static, weight-balanced list of work items
//    (own tile, batch*head): barriers and TMEM are set up once, the TMA producer runs ahead across
//    item boundaries, the next item's own tiles are staged in shared memory while the current item
//    is still computing, and the previous item's outputs are converted and stored while the next
//    item's first scores are already being formed;
//  * the item's own operand tiles (K, V, tK, tV or Q, gO, tQ, G) are copied from the staging area into
//    TMEM as packed 16-bit rows (32 columns each) and are the A operand of every score MMA;
//  * the streamed side advances in sub-tiles of 32 rows; the four score accumulators of a sub-tile
//    take 128 TMEM columns and exist twice (buffers 0 / 1);
//  * three warps issue MMAs, each owning fixed accumulator chains (listed at the issuer code); where
//    two accumulators share the A operand and their B tiles are neighbours in shared memory
//    ([Q;tQ], [K;tK], [V;tV]) one N=64 instruction fills both;
//  * two elementwise warpgroups alternate over the sub-tiles (group g owns buffer g): they turn the
//    accumulators into the 16-bit operands (P, A, gtS, gS, written back in place) with packed fp32x2
//    arithmetic and selects instead of branches.
//
// TMEM map (512 columns):  buffer g at 128*g: S | TS | E | FP (32 each) ; OUT0 at 256 (64) ;
// OUT1 at 320 (64) ; own operand slots at 384 + 32*slot.
// Sub-tiles are numbered globally over the CTA's items (index g): stage g % STAGES, buffer g & 1.
// Barriers: loop_full/loop_empty[stage]; s_full[b] (one arrival per score issuer) -> elementwise;
// p_full[b] (128 threads) -> second-stage issuers; loop_empty[stage] (one arrival per second-stage
// issuer) also releases buffer b to the score issuers.  Per item: own_staged (TMA) -> elementwise;
// own_ready (256 threads) -> issuers and producer; done (second-stage issuers) -> elementwise;
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
  static constexpr int STAGES = 6;
  static constexpr int NTHREADS = 384;  // producer warp, 3 issuer warps, 2 x 4 elementwise warps
  static constexpr int N_SCORE_ISSUERS = (OWN_KEYS && HAS_GT) ? 3 : 2;
  static constexpr int N_OUT_ISSUERS = OWN_KEYS ? 2 : 1;
  static constexpr int N_KEY_TILES = HAS_GT ? 4 : 2;
  static constexpr int N_QRY_TILES = 1 + (HAS_GO ? 1 : 0) + (HAS_GT ? 2 : 0);
  static constexpr int N_OWN = OWN_KEYS ? N_KEY_TILES : N_QRY_TILES;
  static constexpr int N_LOOP = OWN_KEYS ? N_QRY_TILES : N_KEY_TILES;
  static constexpr int LOOP_BYTES = BL * D * 2;  // 4 KiB
  static constexpr int OWN_BYTES = OWN * D * 2;  // 16 KiB
  static constexpr int STAGE_BYTES = N_LOOP * LOOP_BYTES;
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  static constexpr int STAGING_BYTES = N_OWN * OWN_BYTES;
  static constexpr int STAT_BYTES = OWN_KEYS ? STAGES * (BL / 2) * 32 : 0;  // two float4 per column pair
  static constexpr int TILE_BYTES = RING_BYTES + STAGING_BYTES;
  // At least 120 KiB so that a second CTA can never share the SM (the CTA allocates all of TMEM).
  static constexpr int SMEM_NEEDED = TILE_BYTES + STAT_BYTES + 512 + 1024;
  static constexpr int SMEM_BYTES = SMEM_NEEDED > 120 * 1024 ? SMEM_NEEDED : 120 * 1024;
  static constexpr int COL_BUF = 128;  // columns per accumulator buffer
  static constexpr int OFF_S = 0, OFF_TS = 32, OFF_E = 64, OFF_FP = HAS_GT ? 96 : 32;
  static constexpr int COL_OUT0 = 256, COL_OUT1 = 320, COL_OWN = 384;
  static constexpr int COLS_ALLOC = 512;
  // Tile slots (TMEM operand slots / staging tiles of the own side, ring tiles of the streamed side).
  // K|tK, V|tV and Q|tQ are neighbours so that one N=64 instruction can take both as its B operand.
  static constexpr int SLOT_K = 0, SLOT_TK = 1, SLOT_V = HAS_GT ? 2 : 1, SLOT_TV = 3;
  static constexpr int SLOT_Q = 0, SLOT_TQ = 1, SLOT_G = 2, SLOT_GO = HAS_GT ? 3 : 1;
};

__device__ __forceinline__ float2 f2(uint32_t a, uint32_t b) { return make_float2(__uint_as_float(a), __uint_as_float(b)); }

// One work item of the persistent loop.
struct BwdItem {
  int bh, b, own0, loop_begin, n_sub;
};

template <typename T, bool OWN_KEYS, bool HAS_GO, bool HAS_GT>
__global__ void __launch_bounds__(384, 1)
bwd_tc5_d64_kernel(const jvpfa_bwd_args a, const __grid_constant__ Bwd64Maps maps, int* status) {
  using C = Bwd64Cfg<OWN_KEYS, HAS_GO, HAS_GT>;
  constexpr int D = 64, OWN = C::OWN, BL = C::BL, STAGES = C::STAGES;

  if (*(volatile int*)status != 0) return;

  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  unsigned char* smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  unsigned char* sLoop = smem;
  unsigned char* sOwn = smem + C::RING_BYTES;                        // staging of the next item's own tiles
  float4* sStat = reinterpret_cast<float4*>(smem + C::TILE_BYTES);  // [STAGES][BL/2][2]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::TILE_BYTES + C::STAT_BYTES);
  uint64_t* loop_full = bars;                // [STAGES]
  uint64_t* loop_empty = bars + STAGES;      // [STAGES]
  uint64_t* s_full = bars + 2 * STAGES;      // [2]
  uint64_t* p_full = s_full + 2;             // [2]
  uint64_t* own_staged = s_full + 4;
  uint64_t* own_ready = s_full + 5;
  uint64_t* done = s_full + 6;
  uint64_t* out_free = s_full + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_full + 8);
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
    return true;
  };
  auto valid_keys = [&](int b) {
    int n_valid = L;
    if (a.mask.kind == JVPFA_MASK_KVLEN) {
      const int n = a.mask.kv_len[b];
      n_valid = n < 0 ? 0 : (n > L ? L : n);
    }
    return n_valid;
  };
  const int k_max = (n_items + G - 1) / G;

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(loop_full + s, 1);
      mbar_init(loop_empty + s, C::N_OUT_ISSUERS);
    }
    for (int g = 0; g < 2; ++g) {
      mbar_init(s_full + g, C::N_SCORE_ISSUERS);
      mbar_init(p_full + g, 128);
    }
    mbar_init(own_staged, 1);
    mbar_init(own_ready, 256);
    mbar_init(done, C::N_OUT_ISSUERS);
    mbar_init(out_free, 256);
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
    int gbase = 0, kact = 0;
    bool ok = true;
    BwdItem it;
    for (int k = 0; ok && k < k_max; ++k) {
      if (!get_item(k, it)) continue;
      if (it.n_sub == 0) continue;
      // Own tiles of this item -> staging area (free once the previous item's rows sit in TMEM).
      if (kact > 0) ok = mbar_wait(own_ready, (kact - 1) & 1, ab, kAbortBwdOwn);
      if (!ok) break;
      if (lane == 0) {
        mbar_expect_tx(own_staged, C::STAGING_BYTES);
        if constexpr (OWN_KEYS) {
          tma_load_3d(sOwn + C::SLOT_K * C::OWN_BYTES, &maps.k, own_staged, 0, it.own0, it.bh);
          tma_load_3d(sOwn + C::SLOT_V * C::OWN_BYTES, &maps.v, own_staged, 0, it.own0, it.bh);
          if constexpr (HAS_GT) {
            tma_load_3d(sOwn + C::SLOT_TK * C::OWN_BYTES, &maps.tk, own_staged, 0, it.own0, it.bh);
            tma_load_3d(sOwn + C::SLOT_TV * C::OWN_BYTES, &maps.tv, own_staged, 0, it.own0, it.bh);
          }
        } else {
          tma_load_3d(sOwn + C::SLOT_Q * C::OWN_BYTES, &maps.q, own_staged, 0, it.own0, it.bh);
          if constexpr (HAS_GO) tma_load_3d(sOwn + C::SLOT_GO * C::OWN_BYTES, &maps.go, own_staged, 0, it.own0, it.bh);
          if constexpr (HAS_GT) {
            tma_load_3d(sOwn + C::SLOT_TQ * C::OWN_BYTES, &maps.tq, own_staged, 0, it.own0, it.bh);
            tma_load_3d(sOwn + C::SLOT_G * C::OWN_BYTES, &maps.g, own_staged, 0, it.own0, it.bh);
          }
        }
      }
      const size_t stat_off = (size_t)it.bh * L;
      for (int s = 0; s < it.n_sub; ++s) {
        const int g = gbase + s;
        const int st = g % STAGES;
        const uint32_t ph = (g / STAGES) & 1;
        if (!mbar_wait(loop_empty + st, ph ^ 1, ab, kAbortBwdLoopEmpty)) {
          ok = false;
          break;
        }
        const int l0 = it.loop_begin + s * BL;
        if constexpr (OWN_KEYS) {
          // One query per lane: negated statistics, stored pairwise for the packed arithmetic.
          const int i = l0 + lane;
          float nlse = -INFINITY, nmu = 0.f, neps = 0.f, nsub = 0.f;
          if (i < L) {
            nlse = -a.lse[stat_off + i];
            float sub = a.delta[stat_off + i];
            if constexpr (HAS_GT) {
              const float mu = a.mu[stat_off + i], eps = a.eps[stat_off + i];
              nmu = -mu;
              neps = -eps;
              sub += a.cterm[stat_off + i] + eps * mu;
            }
            nsub = -sub;
          }
          float* base = reinterpret_cast<float*>(sStat + (st * (BL / 2) + (lane >> 1)) * 2);
          base[(lane & 1)] = nlse;      // float4 A = (-lse0, -lse1, -mu0, -mu1)
          base[2 + (lane & 1)] = nmu;
          base[4 + (lane & 1)] = neps;  // float4 B = (-eps0, -eps1, -sub0, -sub1)
          base[6 + (lane & 1)] = nsub;
          __syncwarp();
        }
        if (lane == 0) {
          unsigned char* base = sLoop + st * C::STAGE_BYTES;
          mbar_expect_tx(loop_full + st, C::STAGE_BYTES);
          if constexpr (OWN_KEYS) {
            tma_load_3d(base + C::SLOT_Q * C::LOOP_BYTES, &maps.q, loop_full + st, 0, l0, it.bh);
            if constexpr (HAS_GO) tma_load_3d(base + C::SLOT_GO * C::LOOP_BYTES, &maps.go, loop_full + st, 0, l0, it.bh);
            if constexpr (HAS_GT) {
              tma_load_3d(base + C::SLOT_TQ * C::LOOP_BYTES, &maps.tq, loop_full + st, 0, l0, it.bh);
              tma_load_3d(base + C::SLOT_G * C::LOOP_BYTES, &maps.g, loop_full + st, 0, l0, it.bh);
            }
          } else {
            tma_load_3d(base + C::SLOT_K * C::LOOP_BYTES, &maps.k, loop_full + st, 0, l0, it.bh);
            tma_load_3d(base + C::SLOT_V * C::LOOP_BYTES, &maps.v, loop_full + st, 0, l0, it.bh);
            if constexpr (HAS_GT) {
              tma_load_3d(base + C::SLOT_TK * C::LOOP_BYTES, &maps.tk, loop_full + st, 0, l0, it.bh);
              tma_load_3d(base + C::SLOT_TV * C::LOOP_BYTES, &maps.tv, loop_full + st, 0, l0, it.bh);
            }
          }
        }
      }
      gbase += it.n_sub;
      ++kact;
    }
  } else if (warp <= 3) {
    // ------------------------------------------------------------------ MMA issuers 0..2
    const int iss = warp - 1;
    // Accumulator chains (every chain belongs to exactly one issuing thread):
    //   own keys    iss0: [S|TS] = K [Q;tQ]^T, TS += tK Q^T      (GO only: S ; second stage dV += P^T gO)
    //               iss1: E = V G^T          ; second stage dV += A^T G (+ P^T gO)
    //               iss2: FP = tV G^T (+ V gO^T) ; second stage dK += gS^T Q + gtS^T tQ
    //   own queries iss0: [S|TS] = Q [K;tK]^T, TS += tQ K^T
    //               iss1: [E|FP] = G [V;tV]^T (+ FP += gO V^T)   (GO only: FP = gO V^T)
    //               iss2: second stage dQ += gS K + gtS tK
    bool has_scores, has_out;
    if constexpr (OWN_KEYS) {
      has_scores = HAS_GT ? true : (iss != 1);
      has_out = HAS_GT ? (iss != 0) : (iss != 1);
    } else {
      has_scores = iss != 2;
      has_out = iss == 2;
    }
    if (lane == 0 && (has_scores || has_out)) {
      constexpr uint32_t idesc_sc = make_idesc(Fmt<T>::kIdesc, OWN, BL, 0, 0);       // 128 x 32 scores
      constexpr uint32_t idesc_sc2 = make_idesc(Fmt<T>::kIdesc, OWN, 2 * BL, 0, 0);  // 128 x 64: two neighbours
      constexpr uint32_t idesc_out = make_idesc(Fmt<T>::kIdesc, OWN, D, 0, 1);       // 128 x 64 outputs
      const uint32_t own_col = tmem + C::COL_OWN;
      // accumulator columns [off, off + 32*(wide ? 2 : 1)) of buffer buf (+)= own slot (A, TMEM) x
      // streamed tile(s)^T (B, K-major; wide: the tile in b_tile and its neighbour, 64 rows)
      auto score = [&](int buf, int off, int slot, uint32_t b_tile, bool first, bool wide) {
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
          umma_ts(tmem + buf * C::COL_BUF + off, own_col + slot * 32 + ks * 8,
                  make_smem_desc(b_tile + ks * 32, 16, 1024), wide ? idesc_sc2 : idesc_sc, (!first || ks > 0));
      };
      // out (+)= packed operand (A, TMEM, 16 columns) x streamed tile (B, MN-major, 32 rows)
      auto outer = [&](int out_col, int buf, int off, uint32_t b_tile, bool accumulate) {
#pragma unroll
        for (int kk = 0; kk < BL / 16; ++kk)
          umma_ts(tmem + out_col, tmem + buf * C::COL_BUF + off + kk * 8,
                  make_smem_desc(b_tile + kk * 2048, 16, 1024), idesc_out, (accumulate || kk > 0));
      };
      // Scores of global sub-tile g for the accumulators this issuer owns.
      auto issue_scores = [&](int g) -> bool {
        const int st = g % STAGES, buf = g & 1;
        // Buffer `buf` may be overwritten once every second-stage chain of sub-tile g-2 has read it:
        // that is what loop_empty[stage of g-2] records (one arrival per second-stage issuer).
        if (g >= 2 && !mbar_wait(loop_empty + ((g - 2) % STAGES), ((g - 2) / STAGES) & 1, ab, kAbortAux)) return false;
        if (!mbar_wait(loop_full + st, (g / STAGES) & 1, ab, kAbortBwdLoopFull)) return false;
        tc_fence_after();
        const uint32_t lp = smem_u32(sLoop + st * C::STAGE_BYTES);
        auto lt = [&](int slot) { return lp + slot * C::LOOP_BYTES; };
        if constexpr (OWN_KEYS) {
          if (iss == 0) {
            if constexpr (HAS_GT) {
              score(buf, C::OFF_S, C::SLOT_K, lt(C::SLOT_Q), true, true);      // [S|TS] = K [Q;tQ]^T
              score(buf, C::OFF_TS, C::SLOT_TK, lt(C::SLOT_Q), false, false);  // TS += tK Q^T
            } else {
              score(buf, C::OFF_S, C::SLOT_K, lt(C::SLOT_Q), true, false);
            }
          } else if (iss == 1) {
            if constexpr (HAS_GT) score(buf, C::OFF_E, C::SLOT_V, lt(C::SLOT_G), true, false);
          } else {
            if constexpr (HAS_GT) {
              score(buf, C::OFF_FP, C::SLOT_TV, lt(C::SLOT_G), true, false);
              if constexpr (HAS_GO) score(buf, C::OFF_FP, C::SLOT_V, lt(C::SLOT_GO), false, false);
            } else {
              score(buf, C::OFF_FP, C::SLOT_V, lt(C::SLOT_GO), true, false);
            }
          }
        } else {
          if (iss == 0) {
            if constexpr (HAS_GT) {
              score(buf, C::OFF_S, C::SLOT_Q, lt(C::SLOT_K), true, true);      // [S|TS] = Q [K;tK]^T
              score(buf, C::OFF_TS, C::SLOT_TQ, lt(C::SLOT_K), false, false);  // TS += tQ K^T
            } else {
              score(buf, C::OFF_S, C::SLOT_Q, lt(C::SLOT_K), true, false);
            }
          } else {
            if constexpr (HAS_GT) {
              score(buf, C::OFF_E, C::SLOT_G, lt(C::SLOT_V), true, true);      // [E|FP] = G [V;tV]^T
              if constexpr (HAS_GO) score(buf, C::OFF_FP, C::SLOT_GO, lt(C::SLOT_V), false, false);
            } else {
              score(buf, C::OFF_FP, C::SLOT_GO, lt(C::SLOT_V), true, false);
            }
          }
        }
        tc_commit(s_full + buf);
        return true;
      };
      int gbase = 0, kact = 0;
      bool ok = true;
      BwdItem it;
      for (int k = 0; ok && k < k_max; ++k) {
        if (!get_item(k, it)) continue;
        if (it.n_sub == 0) continue;
        ok = mbar_wait(own_ready, kact & 1, ab, kAbortBwdOwn);  // this item's own rows are in TMEM
        if (!ok) break;
        tc_fence_after();
        if (has_scores)
          for (int s = 0; ok && s < 2 && s < it.n_sub; ++s) ok = issue_scores(gbase + s);
        for (int s = 0; ok && s < it.n_sub; ++s) {
          const int g = gbase + s;
          const int st = g % STAGES, buf = g & 1;
          if (has_out) {
            if (!mbar_wait(p_full + buf, (g >> 1) & 1, ab, kAbortBwdPFull)) {
              ok = false;
              break;
            }
            // The first sub-tile overwrites the output accumulators: the previous item's epilogue
            // must have read them.
            if (s == 0 && kact > 0 && !mbar_wait(out_free, (kact - 1) & 1, ab, kAbortBwdDone)) {
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t lp = smem_u32(sLoop + st * C::STAGE_BYTES);
            auto lt = [&](int slot) { return lp + slot * C::LOOP_BYTES; };
            const bool acc = s > 0;
            if constexpr (OWN_KEYS) {
              if (iss == 2) {
                outer(C::COL_OUT0, buf, C::OFF_FP, lt(C::SLOT_Q), acc);                            // dK += gS^T Q
                if constexpr (HAS_GT) outer(C::COL_OUT0, buf, C::OFF_E, lt(C::SLOT_TQ), true);    // dK += gtS^T tQ
              } else if constexpr (HAS_GT) {
                outer(C::COL_OUT1, buf, C::OFF_TS, lt(C::SLOT_G), acc);                            // dV += A^T G
                if constexpr (HAS_GO) outer(C::COL_OUT1, buf, C::OFF_S, lt(C::SLOT_GO), true);    // dV += P^T gO
              } else {
                outer(C::COL_OUT1, buf, C::OFF_S, lt(C::SLOT_GO), acc);                            // dV += P^T gO
              }
            } else {
              outer(C::COL_OUT0, buf, C::OFF_FP, lt(C::SLOT_K), acc);                              // dQ += gS K
              if constexpr (HAS_GT) outer(C::COL_OUT0, buf, C::OFF_E, lt(C::SLOT_TK), true);      // dQ += gtS tK
            }
            tc_commit(loop_empty + st);
          }
          if (has_scores && s + 2 < it.n_sub) ok = issue_scores(g + 2);
        }
        if (ok && has_out) tc_commit(done);
        gbase += it.n_sub;
        ++kact;
      }
    }
  } else {
    // ------------------------------------------------------------------ elementwise warpgroups
    const int wg = (warp - 4) >> 2;  // 0 / 1: accumulator buffer this group works on
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t tbase = tmem + lane_off;
    const uint32_t tbuf = tbase + wg * C::COL_BUF;
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

      // ---- own operand rows: staging area (128-byte-swizzled TMA tiles) -> TMEM, packed 16-bit ----
      if (!mbar_wait(own_staged, kact & 1, ab, kAbortBwdOwn)) {
        alive = false;
        break;
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int slot = 2 * j + wg;
        if (slot < C::N_OWN) {
          uint32_t r[32];
          const unsigned char* src = sOwn + slot * C::OWN_BYTES + row * 128;
#pragma unroll
          for (int x = 0; x < 8; ++x) {
            const uint4 v = *reinterpret_cast<const uint4*>(src + ((x ^ (row & 7)) << 4));
            r[4 * x] = v.x, r[4 * x + 1] = v.y, r[4 * x + 2] = v.z, r[4 * x + 3] = v.w;
          }
          tmem_st32(tbase + C::COL_OWN + slot * 32, r);
        }
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(own_ready);

      // own-queries variant: row statistics, negated
      float r_nlse = -INFINITY, r_nmu = 0.f, r_neps = 0.f, r_nsub = 0.f;
      if constexpr (!OWN_KEYS) {
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
        const int st = g % STAGES;
        const int l0 = it.loop_begin + s * BL;
        if constexpr (OWN_KEYS) {
          if (!mbar_wait(loop_full + st, (g / STAGES) & 1, ab, kAbortBwdLoopFull)) {
            alive = false;
            break;
          }
        }
        if (!mbar_wait(s_full + wg, (g >> 1) & 1, ab, kAbortBwdSFull)) {
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
        uint32_t sv[2][16], fp[2][16];
        uint32_t ts[HAS_GT ? 2 : 1][16], ev[HAS_GT ? 2 : 1][16];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          tmem_ld16(tbuf + C::OFF_S + 16 * c, sv[c]);
          tmem_ld16(tbuf + C::OFF_FP + 16 * c, fp[c]);
          if constexpr (HAS_GT) {
            tmem_ld16(tbuf + C::OFF_TS + 16 * c, ts[c]);
            tmem_ld16(tbuf + C::OFF_E + 16 * c, ev[c]);
          }
        }
        tmem_wait_ld();
        const float4* stat = sStat + st * (BL / 2) * 2;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t pk_gs[8], pk_gt[8], pk_av[8], pk_p[8];
#pragma unroll
          for (int x = 0; x < 8; ++x) {
            const int col = 16 * c + 2 * x;  // even column of the pair
            float2 nl, nmu, neps, nsub;
            if constexpr (OWN_KEYS) {
              const float4 sa = stat[(col >> 1) * 2], sb = stat[(col >> 1) * 2 + 1];
              nl = make_float2(sa.x, sa.y), nmu = make_float2(sa.z, sa.w);
              neps = make_float2(sb.x, sb.y), nsub = make_float2(sb.z, sb.w);
            } else {
              nl = make_float2(r_nlse, r_nlse), nmu = make_float2(r_nmu, r_nmu);
              neps = make_float2(r_neps, r_neps), nsub = make_float2(r_nsub, r_nsub);
            }
            const float2 xs = __ffma2_rn(f2(sv[c][2 * x], sv[c][2 * x + 1]), c2, nl);
            float2 p;
            p.x = (col >= col_lo && col < col_hi) ? fast_exp2(xs.x) : 0.f;
            p.y = (col + 1 >= col_lo && col + 1 < col_hi) ? fast_exp2(xs.y) : 0.f;
            if constexpr (HAS_GT) {
              const float2 tm = __ffma2_rn(f2(ts[c][2 * x], ts[c][2 * x + 1]), sc2, nmu);
              const float2 eb = __fadd2_rn(f2(ev[c][2 * x], ev[c][2 * x + 1]), neps);
              const float2 av = __fmul2_rn(p, tm);
              const float2 gt = __fmul2_rn(p, eb);
              const float2 u = __fadd2_rn(f2(fp[c][2 * x], fp[c][2 * x + 1]), nsub);
              const float2 gs = __fmul2_rn(p, __ffma2_rn(eb, tm, u));
              pk_gs[x] = Elem<T>::pack(gs.x, gs.y);
              pk_gt[x] = Elem<T>::pack(gt.x, gt.y);
              pk_av[x] = Elem<T>::pack(av.x, av.y);
            } else {
              const float2 u = __fadd2_rn(f2(fp[c][2 * x], fp[c][2 * x + 1]), nsub);
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
        mbar_arrive(p_full + wg);
      }
      if (!alive) break;

      // ---- item epilogue: read this group's half of the output accumulators, release them, store ----
      if (!mbar_wait(done, kact & 1, ab, kAbortBwdDone)) {
        alive = false;
        break;
      }
      tc_fence_after();
      {
        uint32_t r0[32];
        uint32_t r1[OWN_KEYS ? 32 : 1];
        tmem_ld32(tbase + C::COL_OUT0 + 32 * wg, r0);
        if constexpr (OWN_KEYS) tmem_ld32(tbase + C::COL_OUT1 + 32 * wg, r1);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(out_free);
        if constexpr (OWN_KEYS) {
          store_half(a.dk, it.bh, own_idx, r0, a.sm_scale);
          store_half(a.dv, it.bh, own_idx, r1, 1.f);
        } else {
          store_half(a.dq, it.bh, own_idx, r0, a.sm_scale);
        }
      }
      gbase += it.n_sub;
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

template <typename T, bool OWN_KEYS, bool HAS_GO, bool HAS_GT>
static int launch_half64(const jvpfa_bwd_args& a, cudaStream_t stream, int* status) {
  using C = Bwd64Cfg<OWN_KEYS, HAS_GO, HAS_GT>;
  Bwd64Maps m;
  const long long BH = (long long)a.B * a.H;
  const CUtensorMapDataType dt = Fmt<T>::kTma;
  const int key_rows = OWN_KEYS ? C::OWN : C::BL;
  const int qry_rows = OWN_KEYS ? C::BL : C::OWN;
  bool ok = encode_map(&m.k, dt, a.k, 64, a.L, BH, key_rows) && encode_map(&m.v, dt, a.v, 64, a.L, BH, key_rows) &&
            encode_map(&m.q, dt, a.q, 64, a.L, BH, qry_rows);
  m.tk = m.tv = m.k;
  m.go = m.tq = m.g = m.q;
  if (HAS_GO) ok = ok && encode_map(&m.go, dt, a.go, 64, a.L, BH, qry_rows);
  if (HAS_GT)
    ok = ok && encode_map(&m.tk, dt, a.tk, 64, a.L, BH, key_rows) && encode_map(&m.tv, dt, a.tv, 64, a.L, BH, key_rows) &&
         encode_map(&m.tq, dt, a.tq, 64, a.L, BH, qry_rows) && encode_map(&m.g, dt, a.gto, 64, a.L, BH, qry_rows);
  if (!ok) {
    set_last_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled(bwd d64)");
    return JVPFA_ERR_CUDA;
  }
  const int sms = sm_count_of_current_device();
  if (sms <= 0) {
    set_last_cuda_error(cudaErrorUnknown, "multiprocessor count");
    return JVPFA_ERR_CUDA;
  }
  auto kern = bwd_tc5_d64_kernel<T, OWN_KEYS, HAS_GO, HAS_GT>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
  if (e != cudaSuccess) {
    set_last_cuda_error(e, "cudaFuncSetAttribute(bwd_tc5_d64)");
    return JVPFA_ERR_CUDA;
  }
  const long long n_items = (long long)((a.L + C::OWN - 1) / C::OWN) * BH;
  const int grid = (int)(n_items < sms ? n_items : sms);
  kern<<<grid, C::NTHREADS, C::SMEM_BYTES, stream>>>(a, m, status);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_cuda_error(e, "launch bwd_tc5_d64");
    return JVPFA_ERR_CUDA;
  }
  return JVPFA_OK;
}

template <typename T, bool HAS_GO, bool HAS_GT>
static int launch_both64(const jvpfa_bwd_args& a, cudaStream_t s) {
  int* status = tc5_status_device_ptr();
  if (!status) {
    set_last_cuda_error(cudaErrorUnknown, "status word address");
    return JVPFA_ERR_CUDA;
  }
  int rc = JVPFA_OK;
  if (!(a.impl & JVPFA_IMPL_ONLY_DQ)) rc = launch_half64<T, true, HAS_GO, HAS_GT>(a, s, status);
  if (rc) return rc;
  if (!(a.impl & JVPFA_IMPL_ONLY_DKDV)) rc = launch_half64<T, false, HAS_GO, HAS_GT>(a, s, status);
  return rc;
}

template <typename T>
static int launch_t64(const jvpfa_bwd_args& a, cudaStream_t s) {
  const bool go = a.go != nullptr, gt = a.gto != nullptr;
  if (go && gt) return launch_both64<T, true, true>(a, s);
  if (gt) return launch_both64<T, false, true>(a, s);
  return launch_both64<T, true, false>(a, s);
}

}  // namespace tc5

int launch_bwd_tc5_d64(const jvpfa_bwd_args& a, cudaStream_t s) {
  return a.dtype == JVPFA_BF16 ? tc5::launch_t64<__nv_bfloat16>(a, s) : tc5::launch_t64<__half>(a, s);
}

}  // namespace jvpfa
