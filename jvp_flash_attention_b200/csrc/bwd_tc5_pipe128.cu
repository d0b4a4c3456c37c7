// Backward of <gO, O> + <gtO, tO> for head dimension 128, bf16 / fp16, on the Blackwell tensor cores, with the score
// products of the next tile running under the elementwise work of the current one.
//
// Same split as the register-tiled backward (bwd_generic.cu; upstream jvp_attention.py:2008-2233): one launch owns
// 128-key tiles and loops over queries (dK, dV), one owns 128-query tiles and loops over keys (dQ).  Both are
// instances of one template:
//   "own" side  : 128 rows, one per TMEM lane; four operand tiles resident in smem
//                 own keys: K, tK, V, tV        own queries: Q, tQ, G, gO        (G = cotangent of tO)
//   "loop" side : tiles of BL rows (32 with own keys, 48 with own queries) streamed by TMA, the tensors of a stage
//                 adjacent.  Own keys: Q, tQ, G, gO in one three-stage ring.  Own queries: K, tK in a three-stage
//                 ring (the output products read them again), V, tV in a one-stage ring that comes free as soon
//                 as the tile's scores exist.
// TMEM: two buffers of four 128 x BL fp32 score accumulators [S | TS | E | FP], then the outputs (dK | dV, or dQ).
// Per loop tile the MMA warp forms
//     [S | TS] = own0 [loop0 | loop1]^T ,  TS += own1 loop0^T     (scores and tangent scores)
//     [E | FP] = own2 [loop2 | loop3]^T ,  FP += own3 loop2^T     (own keys: E = V G^T, FP = V gO^T + tV G^T)
// where products that share the 128-row operand are one instruction over the adjacent loop tiles.  The elementwise
// threads (BL / 16 warpgroups, 16 columns each) read the four accumulators and write the 16-bit operands
//     P, A = P*(tS-mu), gtS = P*(E-eps), gS = P*((E-eps)*(tS-mu) + FP - delta - cterm - eps*mu)
// back over the columns they have just read: warpgroup h puts its 16 columns of gS and gtS over its half of S and
// its A and P over its half of TS, so that neither group can overwrite what the other still has to read.  A second
// group of MMAs (A operand from TMEM, one contraction step per 16-column piece; B = the streamed tiles used
// MN-major) accumulates
//     dK += gS Q + gtS tQ ,  dV += A G + P gO      or      dQ += gS K + gtS tK.
// The issuer's order is  scores(0), scores(1), out(0), scores(2), out(1), ...: the tensor pipe executes in issue
// order, so scores(t+2) overwrites buffer t & 1 only after out(t) has read its operands from it.
// Formulas: see bwd_generic.cu.  All waits are bounded (tc5_common.cuh); after one that gave up the CTA's output
// rows carry NaN.
#include "tc5_common.cuh"

namespace jvpfa {
namespace tc5 {

struct BwdPipeMaps {
  CUtensorMap k, v, tk, tv;   // key-side tensors
  CUtensorMap q, go, tq, g;   // query-side tensors (g = cotangent of tO)
};

template <bool OWN_KEYS, bool HAS_GO, bool HAS_GT>
struct BwdPipeCfg {
  static constexpr int D = 128;
  static constexpr int OWN = 128;
  // Rows of a loop tile.  An MMA instruction costs about 58 cycles whatever its N up to 64, so wider tiles mean fewer
  // instructions per column.  Own keys: dK | dV take 256 TMEM columns, which leaves two score buffers of 4 x 32; own
  // queries: dQ takes 128, which leaves two buffers of 4 x 48.
  static constexpr int BL = OWN_KEYS ? 32 : 48;
  static constexpr int NP = BL / 16;                // 16-column pieces = elementwise warpgroups
  static constexpr int NTHREADS = 64 + 128 * NP + 32;  // producer, issuer, NP elementwise warpgroups, second issuer
  static constexpr int WARP_ISSUER2 = 2 + 4 * NP;
  static constexpr int OWN_BYTES = OWN * D * 2;     // 32 KiB: two 64-column halves of 16 KiB
  static constexpr int OWN_HALF = OWN * 128;
  static constexpr int LQ_BYTES = BL * 128;         // one loop tensor, one 64-column half
  // Ring X holds the loop tensors that the output products read again (they stay until the tile's outputs are done);
  // ring Y those that only the score products read (free as soon as the scores exist).  Own keys: all four in X.
  static constexpr int NX = OWN_KEYS ? 4 : 2;
  static constexpr int NY = 4 - NX;
  static constexpr int XSTAGES = 3;
  static constexpr int X_HALF = NX * LQ_BYTES;      // [x0 | x1 (| x2 | x3)] of one half
  static constexpr int X_STAGE = 2 * X_HALF;
  static constexpr int Y_HALF = NY * LQ_BYTES;
  static constexpr int Y_STAGE = 2 * Y_HALF;        // one stage
  static constexpr int OFF_X = 4 * OWN_BYTES;
  static constexpr int OFF_Y = OFF_X + XSTAGES * X_STAGE;
  static constexpr int TILE_BYTES = OFF_Y + Y_STAGE;  // 224 KiB
  static constexpr int STAT_BYTES = OWN_KEYS ? XSTAGES * BL * 16 : 0;
  static constexpr int SMEM_BYTES = TILE_BYTES + STAT_BYTES + 256 + 1024;
  // tensors actually loaded
  static constexpr int N_KEY = HAS_GT ? 4 : 2;                               // K, V (+ tK, tV)
  static constexpr int N_QRY = 1 + (HAS_GO ? 1 : 0) + (HAS_GT ? 2 : 0);      // Q (+ gO) (+ tQ, G)
  static constexpr int N_OWN = OWN_KEYS ? N_KEY : N_QRY;
  static constexpr int N_X = OWN_KEYS ? N_QRY : (HAS_GT ? 2 : 1);            // own queries: K (+ tK)
  static constexpr int N_Y = OWN_KEYS ? 0 : (HAS_GT ? 2 : 1);                // own queries: V (+ tV)
  // TMEM columns
  static constexpr int SC_COLS = 4 * BL;  // one buffer: S | TS | E | FP
  static constexpr int COL_S = 0, COL_TS = BL, COL_E = 2 * BL, COL_FP = 3 * BL;
  // Packed operands: piece h (columns 16h .. 16h+15 of the tile) of gS at COL_S + 16h, of gtS 8 columns on;
  // of A at COL_TS + 16h, of P 8 columns on.
  static constexpr int COL_OUT0 = 2 * SC_COLS;
  static constexpr int COL_OUT1 = COL_OUT0 + D;
  static constexpr int COLS_ALLOC = 512;
  static_assert(COL_OUT0 + (OWN_KEYS ? 2 : 1) * D <= 512, "TMEM budget");
};
static_assert(BwdPipeCfg<true, true, true>::SMEM_BYTES <= 227 * 1024, "shared memory budget");
static_assert(BwdPipeCfg<false, true, true>::SMEM_BYTES <= 227 * 1024, "shared memory budget");

// MK == 3: walks the loop tiles of a CTA that hold a true mask entry, in order.  The bitmaps of jvpfa_mask_tiles have one
// bit per 128-query x 64-key tile.  Own keys: w points at the transposed bitmap's entry of the own 128-key tile (bit =
// 128-query tile, four 32-row loop tiles each).  Own queries: w points at the bitmap's entry of the own 128-query tile
// (bit = 64-key tile); a 48-key loop tile is live if one of the one or two 64-key tiles it overlaps is.
template <bool OWN_KEYS, int BL>
struct LoopWalk {
  const unsigned long long* w = nullptr;
  int n_cand = 0, n_bits = 1, c = 0;
  bool rows = true;  // false: the mask has one row for all queries
  __device__ __forceinline__ bool bit(int b) const { return (__ldg(w + (b >> 6)) >> (b & 63)) & 1ull; }
  __device__ __forceinline__ bool live(int cc) const {
    if constexpr (OWN_KEYS) {
      return bit(rows ? (cc * BL) >> 7 : 0);
    } else {
      const int lo = (cc * BL) >> 6, hi = min((cc * BL + BL - 1) >> 6, n_bits - 1);
      return bit(lo) || bit(hi);
    }
  }
  __device__ __forceinline__ int next() {  // index of the next live loop tile (the caller asks no more often than there are)
    while (c < n_cand && !live(c)) ++c;
    return c++;
  }
  __device__ __forceinline__ int count() const {
    int n = 0;
    for (int cc = 0; cc < n_cand; ++cc) n += live(cc) ? 1 : 0;
    return n;
  }
};

// MK: 0 = none / causal / key padding; 1 = uint8 mask; 2 = bias of the element type T; 3 = uint8 mask with the tile
// bitmaps (loop tiles without a true entry are not visited).  For 1 and 2 every elementwise
// thread fetches the 16 mask elements of its piece of the tile from global memory before it waits for the scores (own
// queries: one or two 16-byte loads of the thread's mask row; own keys: one element of each of 16 query rows, the lanes
// of a warp reading neighbouring keys).  Key stride 1, 16-byte aligned rows and L % 16 == 0 are the host's
// responsibility.
template <typename T, bool OWN_KEYS, bool HAS_GO, bool HAS_GT, int MK>
__global__ void __launch_bounds__(BwdPipeCfg<OWN_KEYS, HAS_GO, HAS_GT>::NTHREADS, 1)
bwd_tc5_pipe128_kernel(const jvpfa_bwd_args a, const __grid_constant__ BwdPipeMaps maps, int* status) {
  using C = BwdPipeCfg<OWN_KEYS, HAS_GO, HAS_GT>;
  constexpr int D = C::D, OWN = C::OWN, BL = C::BL, STAGES = C::XSTAGES, NP = C::NP;

  // The own-queries launch that follows reads nothing this kernel writes: it is launched with programmatic
  // stream serialization and fills the SMs as this kernel's last CTAs leave them.
  if constexpr (OWN_KEYS) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const bool dead_on_entry = *(volatile int*)status != 0;  // an earlier bounded wait gave up

  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  unsigned char* smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  unsigned char* sOwn = smem;
  unsigned char* sX = smem + C::OFF_X;
  unsigned char* sY = smem + C::OFF_Y;
  float4* sStat = reinterpret_cast<float4*>(smem + C::TILE_BYTES);  // OWN_KEYS: [STAGES][BL] {lse, mu, eps, sub}
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::TILE_BYTES + C::STAT_BYTES);
  uint64_t* own_full = bars + 0;
  uint64_t* loop_full = bars + 1;   // [3]
  uint64_t* loop_empty = bars + 4;  // [3]
  uint64_t* s_full = bars + 7;      // [2]
  uint64_t* p_full = bars + 9;      // [2]
  uint64_t* done = bars + 11;
  uint64_t* y_full = bars + 12;   // ring Y (one stage)
  uint64_t* y_empty = bars + 13;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* n_live = reinterpret_cast<int*>(tmem_slot + 2);  // MK == 3: live loop tiles of this CTA

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int L = a.L;
  const int bh = blockIdx.y;
  const int tma_b = bh / a.H, tma_h = bh - tma_b * a.H;  // coordinates in the (D, L, H, B) tensor maps
  const bool causal = a.mask.kind == JVPFA_MASK_CAUSAL;
  int n_valid = L;
  if (a.mask.kind == JVPFA_MASK_KVLEN) {
    const int n = a.mask.kv_len[tma_b];
    n_valid = n < 0 ? 0 : (n > L ? L : n);
  }
  // Tile ranges.  Own keys: heaviest (lowest) key tiles come first by construction; own queries: reversed so that
  // the heaviest (highest) query tiles start first.
  int own0, loop_begin, n_tiles;
  if constexpr (OWN_KEYS) {
    own0 = blockIdx.x * OWN;
    loop_begin = causal ? own0 : 0;
    n_tiles = (L - loop_begin + BL - 1) / BL;
    if (own0 >= n_valid) n_tiles = 0;
  } else {
    own0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * OWN;
    loop_begin = 0;
    int n_end = n_valid;
    if (causal) n_end = min(n_end, own0 + OWN);
    n_tiles = (n_end + BL - 1) / BL;
  }
  const size_t stat_off = (size_t)bh * L;
  LoopWalk<OWN_KEYS, BL> walk0;
  if constexpr (MK == 3) {
    // the bitmaps have the mask's own extents: a broadcast dimension (stride 0) has one entry
    const long long hm = (a.mask.stride[0] ? (long long)tma_b * (a.mask.stride[1] ? a.H : 1) : 0) +
                         (a.mask.stride[1] ? tma_h : 0);
    const int n_t128 = (L + 127) / 128;
    walk0.rows = a.mask.stride[2] != 0;
    walk0.n_cand = n_tiles;
    if constexpr (OWN_KEYS) {
      const int n_words_t = walk0.rows ? (n_t128 + 63) / 64 : 1;
      walk0.w = reinterpret_cast<const unsigned long long*>(a.mask_tile_live_t) + (hm * n_t128 + own0 / OWN) * n_words_t;
    } else {
      walk0.n_bits = (L + 63) / 64;
      const int n_words = (walk0.n_bits + 63) / 64;
      walk0.w = reinterpret_cast<const unsigned long long*>(a.mask_tile_live) +
                (walk0.rows ? hm * n_t128 + own0 / OWN : hm) * n_words;
    }
  }

  // NaN into this CTA's output rows: the results of this launch are not to be trusted
  auto poison = [&]() {
    if (tid < OWN && own0 + tid < L) {
      if constexpr (OWN_KEYS) {
        poison_row<T>(a.dk, stat_off + own0 + tid, D);
        poison_row<T>(a.dv, stat_off + own0 + tid, D);
      } else {
        poison_row<T>(a.dq, stat_off + own0 + tid, D);
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
    mbar_init(own_full, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(loop_full + s, OWN_KEYS ? 2 : 1);  // TMA bytes (+ the row statistics, own keys)
      mbar_init(loop_empty + s, OWN_KEYS ? 2 : 1);  // own keys: both issuing threads read the stage
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(s_full + s, 2);  // one commit per issuing thread
      mbar_init(p_full + s, 128 * NP);
    }
    mbar_init(done, 1);
    mbar_init(y_full, 1);
    mbar_init(y_empty, 1);
    *abort_flag = 0;
    fence_mbar_init();
    if constexpr (MK == 3) *n_live = walk0.count();
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
  if constexpr (MK == 3) n_tiles = *n_live;

  // Tensor map of own slot s / loop slot s (nullptr: the slot is not used by this instance).
  auto own_map = [&](int s) -> const CUtensorMap* {
    if constexpr (OWN_KEYS) {
      if (s == 0) return &maps.k;
      if (s == 2) return &maps.v;
      if (!HAS_GT) return nullptr;
      return s == 1 ? &maps.tk : &maps.tv;
    } else {
      if (s == 0) return &maps.q;
      if (s == 3) return HAS_GO ? &maps.go : nullptr;
      if (!HAS_GT) return nullptr;
      return s == 1 ? &maps.tq : &maps.g;
    }
  };
  // Tensor map of slot s of ring X / ring Y (nullptr: not used by this instance).
  auto x_map = [&](int s) -> const CUtensorMap* {
    if constexpr (OWN_KEYS) {  // Q, tQ, G, gO
      if (s == 0) return &maps.q;
      if (s == 3) return HAS_GO ? &maps.go : nullptr;
      if (!HAS_GT) return nullptr;
      return s == 1 ? &maps.tq : &maps.g;
    } else {  // K, tK
      if (s == 0) return &maps.k;
      return (s == 1 && HAS_GT) ? &maps.tk : nullptr;
    }
  };
  auto y_map = [&](int s) -> const CUtensorMap* {  // own queries: V, tV
    if (OWN_KEYS) return nullptr;
    if (s == 0) return &maps.v;
    return (s == 1 && HAS_GT) ? &maps.tv : nullptr;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (+ stats)
    if (n_tiles > 0) {
      if (lane == 0) {
        mbar_expect_tx(own_full, C::N_OWN * C::OWN_BYTES);
#pragma unroll
        for (int s = 0; s < 4; ++s) {
          const CUtensorMap* m = own_map(s);
          if (m == nullptr) continue;
          for (int hf = 0; hf < 2; ++hf)
            tma_load_4d(sOwn + s * C::OWN_BYTES + hf * C::OWN_HALF, m, own_full, hf * 64, own0, tma_h, tma_b);
        }
      }
      auto walk = walk0;
      for (int t = 0; t < n_tiles; ++t) {
        const int st = t % STAGES;
        const uint32_t ph = (t / STAGES) & 1;
        if (!mbar_wait(loop_empty + st, ph ^ 1, ab, kAbortBwdLoopEmpty)) break;
        const int l0 = MK == 3 ? walk.next() * BL : loop_begin + t * BL;
        if (lane == 0) {
          unsigned char* base = sX + st * C::X_STAGE;
          mbar_expect_tx(loop_full + st, C::N_X * 2 * C::LQ_BYTES);
#pragma unroll
          for (int s = 0; s < C::NX; ++s) {
            const CUtensorMap* m = x_map(s);
            if (m == nullptr) continue;
            for (int hf = 0; hf < 2; ++hf)
              tma_load_4d(base + hf * C::X_HALF + s * C::LQ_BYTES, m, loop_full + st, hf * 64, l0, tma_h, tma_b);
          }
        }
        if constexpr (C::NY > 0) {
          // ring Y comes free (scores of the previous tile) after the X stage did (outputs of three tiles ago)
          if (!mbar_wait(y_empty, (t & 1) ^ 1, ab, kAbortBwdLoopEmpty)) break;
          if (lane == 0) {
            mbar_expect_tx(y_full, C::N_Y * 2 * C::LQ_BYTES);
#pragma unroll
            for (int s = 0; s < C::NY; ++s) {
              const CUtensorMap* m = y_map(s);
              if (m == nullptr) continue;
              for (int hf = 0; hf < 2; ++hf)
                tma_load_4d(sY + hf * C::Y_HALF + s * C::LQ_BYTES, m, y_full, hf * 64, l0, tma_h, tma_b);
            }
          }
        }
        if constexpr (OWN_KEYS) {
          // per-query statistics of this tile, combined once for all 128 key rows; fetched after the tile
          // loads have been issued, so that the two latencies overlap
          {
            const int i = l0 + lane;
            float4 s4 = make_float4(INFINITY, 0.f, 0.f, 0.f);
            if (i < L) {
              s4.x = a.lse[stat_off + i];
              s4.w = a.delta[stat_off + i];
              if constexpr (HAS_GT) {
                s4.y = a.mu[stat_off + i];
                s4.z = a.eps[stat_off + i];
                s4.w += a.cterm[stat_off + i] + s4.z * s4.y;
              }
            }
            sStat[st * BL + lane] = s4;
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(loop_full + st);  // second arrival: the statistics are in place
        }
      }
    }
  } else if (warp == 1 || warp == C::WARP_ISSUER2) {
    // ------------------------------------------------------------------ MMA issuers
    // One thread cannot issue an MMA more often than about every 58 cycles, whatever its shape; two threads together
    // can.  The first issuer forms [S | TS] and, after the elementwise threads, the outputs; the second forms [E | FP].
    // Everything that reads what the elementwise threads write (they write over S and TS only) is issued by the first
    // thread, after that thread's own scores into the same buffer two tiles earlier and before its next ones: the
    // tensor pipe keeps one thread's instructions in order, so no barrier between the two issuers is needed.  The
    // second thread waits for p_full(t) only to know that E and FP of tile t have been read before it overwrites them.
    if (lane == 0 && n_tiles > 0) {
      const bool second = warp != 1;
      constexpr uint32_t idesc_n1 = make_idesc(Fmt<T>::kIdesc, OWN, BL, 0, 0);      // one 128 x BL accumulator
      constexpr uint32_t idesc_n2 = make_idesc(Fmt<T>::kIdesc, OWN, 2 * BL, 0, 0);  // two adjacent accumulators
      constexpr uint32_t idesc_out = make_idesc(Fmt<T>::kIdesc, OWN, D, 0, 1);      // 128 x 128 outputs
      // Shared-memory descriptors as low words (tc5_common.cuh): the high word is the same for every tile used here,
      // and stepping through a tile is an integer add.  K-major operands: contraction step ks over the head dimension
      // = 32 bytes inside a 64-column half, the halves OWN_HALF / X_HALF / Y_HALF apart.  MN-major ring-X tiles (B of the
      // outputs): contraction step kk = 16 rows = 2048 bytes, leading offset = distance of the two 64-column halves.
      const uint32_t a_lo0 = kDescLo | (smem_u32(sOwn) >> 4);
      constexpr uint32_t kMnLo = (uint32_t)(C::X_HALF >> 4) << 16;
      auto a_off = [](int slot, int ks) -> uint32_t {
        return (uint32_t)(slot * C::OWN_BYTES + (ks >> 2) * C::OWN_HALF + (ks & 3) * 32) >> 4;
      };
      auto b_off = [](uint32_t half, int slot, int ks) -> uint32_t {
        return (uint32_t)((ks >> 2) * half + slot * C::LQ_BYTES + (ks & 3) * 32) >> 4;
      };
      // first issuer: [S | TS] = own0 [loop0 | loop1]^T, TS += own1 loop0^T
      auto issue_s = [&](int t) -> bool {
        const int st = t % STAGES;
        if (!mbar_wait(loop_full + st, (t / STAGES) & 1, ab, kAbortBwdLoopFull)) return false;
        tc_fence_after();
        const uint32_t lx = kDescLo | (smem_u32(sX + st * C::X_STAGE) >> 4);
        const uint32_t sc = tmem + (t & 1) * C::SC_COLS;
        constexpr uint32_t id = HAS_GT ? idesc_n2 : idesc_n1;
        umma_ss_lo<false>(sc + C::COL_S, a_lo0 + a_off(0, 0), lx + b_off(C::X_HALF, 0, 0), id);
#pragma unroll
        for (int ks = 1; ks < 8; ++ks)
          umma_ss_lo<true>(sc + C::COL_S, a_lo0 + a_off(0, ks), lx + b_off(C::X_HALF, 0, ks), id);
        if constexpr (HAS_GT) {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            umma_ss_lo<true>(sc + C::COL_TS, a_lo0 + a_off(1, ks), lx + b_off(C::X_HALF, 0, ks), idesc_n1);
        }
        tc_commit(s_full + (t & 1));
        return true;
      };
      // second issuer: [E | FP] = own2 [loop2 | loop3]^T, FP += own3 loop2^T; loop tensors 2 and 3 are slots 2, 3 of the
      // X stage (own keys) or slots 0, 1 of ring Y (own queries)
      auto issue_e = [&](int t) -> bool {
        uint32_t l2;
        if constexpr (OWN_KEYS) {
          const int st = t % STAGES;
          if (!mbar_wait(loop_full + st, (t / STAGES) & 1, ab, kAbortBwdLoopFull)) return false;
          l2 = (kDescLo | (smem_u32(sX + st * C::X_STAGE) >> 4)) + ((2 * C::LQ_BYTES) >> 4);
        } else {
          if (!mbar_wait(y_full, t & 1, ab, kAbortBwdLoopFull)) return false;
          l2 = kDescLo | (smem_u32(sY) >> 4);
        }
        tc_fence_after();
        constexpr uint32_t h2 = OWN_KEYS ? C::X_HALF : C::Y_HALF;
        const uint32_t sc = tmem + (t & 1) * C::SC_COLS;
        if constexpr (HAS_GT) {
          constexpr bool wide = !OWN_KEYS || HAS_GO;  // [E | FP] in one instruction
          umma_ss_lo<false>(sc + C::COL_E, a_lo0 + a_off(2, 0), l2 + b_off(h2, 0, 0), wide ? idesc_n2 : idesc_n1);
#pragma unroll
          for (int ks = 1; ks < 8; ++ks)
            umma_ss_lo<true>(sc + C::COL_E, a_lo0 + a_off(2, ks), l2 + b_off(h2, 0, ks), wide ? idesc_n2 : idesc_n1);
          if constexpr (OWN_KEYS || HAS_GO) {
            umma_ss_lo<wide>(sc + C::COL_FP, a_lo0 + a_off(3, 0), l2 + b_off(h2, 0, 0), idesc_n1);
#pragma unroll
            for (int ks = 1; ks < 8; ++ks)
              umma_ss_lo<true>(sc + C::COL_FP, a_lo0 + a_off(3, ks), l2 + b_off(h2, 0, ks), idesc_n1);
          }
        } else {
          // FP = V gO^T (own keys: own2 loop3^T) or gO V^T (own queries: own3 loop2^T)
          constexpr int fa = OWN_KEYS ? 2 : 3, fb = OWN_KEYS ? 1 : 0;
          umma_ss_lo<false>(sc + C::COL_FP, a_lo0 + a_off(fa, 0), l2 + b_off(h2, fb, 0), idesc_n1);
#pragma unroll
          for (int ks = 1; ks < 8; ++ks)
            umma_ss_lo<true>(sc + C::COL_FP, a_lo0 + a_off(fa, ks), l2 + b_off(h2, fb, ks), idesc_n1);
        }
        if constexpr (OWN_KEYS) tc_commit(loop_empty + (t % STAGES)); else tc_commit(y_empty);
        tc_commit(s_full + (t & 1));
        return true;
      };
      bool ok = mbar_wait(own_full, 0, ab, kAbortBwdOwn);
      if (second) {
        if (ok) ok = issue_e(0);
        for (int t = 0; ok && t + 1 < n_tiles; ++t) {
          if (!issue_e(t + 1)) break;
          if (!mbar_wait(p_full + (t & 1), (t >> 1) & 1, ab, kAbortBwdPFull)) break;
        }
      } else {
        if (ok) ok = issue_s(0);
        for (int t = 0; ok && t < n_tiles; ++t) {
          if (t + 1 < n_tiles && !issue_s(t + 1)) break;
          if (!mbar_wait(p_full + (t & 1), (t >> 1) & 1, ab, kAbortBwdPFull)) break;
          tc_fence_after();
          const int st = t % STAGES;
          const uint32_t mx = kMnLo | (smem_u32(sX + st * C::X_STAGE) >> 4);
          const uint32_t sc = tmem + (t & 1) * C::SC_COLS;
          const uint32_t acc = t > 0;
          // Contraction step kk = NP * term + piece: rows 16 * piece .. of X tile (slot + term), operand piece at
          // column 16 * piece + 8 * term of the accumulator it was written over.
          // dK or dQ += gS x0 + gtS x1
          umma_ts_lo_dyn(tmem + C::COL_OUT0, sc + C::COL_S, mx, idesc_out, acc);
#pragma unroll
          for (int kk = 1; kk < (HAS_GT ? 2 : 1) * NP; ++kk)
            umma_ts_lo<true>(tmem + C::COL_OUT0, sc + C::COL_S + 16 * (kk % NP) + 8 * (kk / NP), mx + kk * 128, idesc_out);
          if constexpr (OWN_KEYS) {
            if constexpr (HAS_GT) {
              // dV += A G + P gO   (X slots 2, 3)
              constexpr uint32_t o2 = (2 * C::LQ_BYTES) >> 4;
              umma_ts_lo_dyn(tmem + C::COL_OUT1, sc + C::COL_TS, mx + o2, idesc_out, acc);
#pragma unroll
              for (int kk = 1; kk < (HAS_GO ? 2 : 1) * NP; ++kk)
                umma_ts_lo<true>(tmem + C::COL_OUT1, sc + C::COL_TS + 16 * (kk % NP) + 8 * (kk / NP), mx + o2 + kk * 128, idesc_out);
            } else {
              // dV += P gO   (X slot 3)
              constexpr uint32_t o3 = (3 * C::LQ_BYTES) >> 4;
              umma_ts_lo_dyn(tmem + C::COL_OUT1, sc + C::COL_TS + 8, mx + o3, idesc_out, acc);
#pragma unroll
              for (int kk = 1; kk < NP; ++kk)
                umma_ts_lo<true>(tmem + C::COL_OUT1, sc + C::COL_TS + 16 * kk + 8, mx + o3 + kk * 128, idesc_out);
            }
          }
          tc_commit(loop_empty + st);
        }
        tc_commit(done);
      }
    }
  } else {
    // ------------------------------------------------------------------ elementwise + epilogue
    const int quarter = warp & 3;       // TMEM lane quarter this warp may access
    const int piece = (warp - 2) >> 2;  // warpgroup: columns 16 * piece .. 16 * piece + 15 of every loop tile
    const int row = quarter * 32 + lane;
    const int own_idx = own0 + row;  // key index (OWN_KEYS) or query index
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t tbase = tmem + lane_off;
    const float scale_log2 = a.sm_scale * kLog2e;
    bool alive = true;

    // own-queries variant: this thread's row statistics
    float r_lse = INFINITY, r_mu = 0.f, r_eps = 0.f, r_sub = 0.f;
    if constexpr (!OWN_KEYS) {
      if (own_idx < L) {
        r_lse = a.lse[stat_off + own_idx];
        r_sub = a.delta[stat_off + own_idx];
        if constexpr (HAS_GT) {
          r_mu = a.mu[stat_off + own_idx];
          r_eps = a.eps[stat_off + own_idx];
          r_sub += a.cterm[stat_off + own_idx] + r_eps * r_mu;
        }
      }
    }

    constexpr bool BOOLM = MK == 1 || MK == 3;
    constexpr int MESZ = BOOLM ? 1 : 2;  // bytes per mask element
    const unsigned char* mbase = nullptr;
    long long mpitch = 0;
    if constexpr (MK != 0) {
      mbase = reinterpret_cast<const unsigned char*>(a.mask.ptr) +
              ((long long)tma_b * a.mask.stride[0] + (long long)tma_h * a.mask.stride[1]) * MESZ;
      mpitch = a.mask.stride[2] * MESZ;
    }

    auto walk = walk0;
    for (int t = 0; t < n_tiles; ++t) {
      const int st = t % STAGES;
      const int l0 = MK == 3 ? walk.next() * BL : loop_begin + t * BL;
      // MK != 0: the piece's 16 mask / bias elements, one per column (indices clamped into the tensor; what lies
      // outside is switched off by the index tests below)
      uint32_t mraw[MK == 0 ? 1 : 16];
      if constexpr (MK != 0) {
        const int c0 = l0 + 16 * piece;  // first loop-side index of this thread's columns
        if constexpr (OWN_KEYS) {
          const unsigned char* pm = mbase + (long long)min(own_idx, L - 1) * MESZ;
#pragma unroll
          for (int x = 0; x < 16; ++x) {
            const unsigned char* el = pm + (long long)min(c0 + x, L - 1) * mpitch;
            mraw[x] = BOOLM ? ldg_nc_u8(el) : ldg_nc_u16(el);
          }
        } else {
          const unsigned char* pm = mbase + (long long)min(own_idx, L - 1) * mpitch + (size_t)c0 * MESZ;
          uint32_t w[4 * MESZ];
#pragma unroll
          for (int j = 0; j < MESZ; ++j) {
            uint4 r = make_uint4(0u, 0u, 0u, 0u);
            if (c0 + (j + 1) * (16 / MESZ) <= L) r = ldg_nc_v4(pm + 16 * j);
            w[4 * j] = r.x, w[4 * j + 1] = r.y, w[4 * j + 2] = r.z, w[4 * j + 3] = r.w;
          }
#pragma unroll
          for (int x = 0; x < 16; ++x)
            mraw[x] = BOOLM ? ((w[x >> 2] >> ((x & 3) * 8)) & 0xffu) : ((w[x >> 1] >> ((x & 1) * 16)) & 0xffffu);
        }
      }
      if constexpr (OWN_KEYS) {
        if (!mbar_wait(loop_full + st, (t / STAGES) & 1, ab, kAbortBwdLoopFull)) {
          alive = false;
          break;
        }
      }
      if (!mbar_wait(s_full + (t & 1), (t >> 1) & 1, ab, kAbortBwdSFull)) {
        alive = false;
        break;
      }
      tc_fence_after();
      const uint32_t sc = tbase + (t & 1) * C::SC_COLS + 16 * piece;
      uint32_t s[16], fp[16];
      uint32_t ts[HAS_GT ? 16 : 1], e[HAS_GT ? 16 : 1];
      tmem_ld16(sc + C::COL_S, s);
      tmem_ld16(sc + C::COL_FP, fp);
      if constexpr (HAS_GT) {
        tmem_ld16(sc + C::COL_TS, ts);
        tmem_ld16(sc + C::COL_E, e);
      }
      tmem_wait_ld();
      // does any element of this tile need the mask test?
      bool partial;
      if constexpr (OWN_KEYS) {
        partial = (own0 + OWN > n_valid) || (causal && own0 + OWN - 1 > l0);
      } else {
        partial = (l0 + BL > n_valid) || (causal && l0 + BL - 1 > own0);
      }
      const float4* stat = sStat + st * BL + 16 * piece;
      uint32_t pk_gs[8], pk_gt[HAS_GT ? 8 : 1], pk_av[(HAS_GT && OWN_KEYS) ? 8 : 1], pk_p[OWN_KEYS ? 8 : 1];
#pragma unroll
      for (int x2 = 0; x2 < 8; ++x2) {
        float pv[2], gs[2], av[2], gt[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int col = 2 * x2 + h;
          float lse, mu, eps, sub;
          int i, j;
          if constexpr (OWN_KEYS) {
            const float4 s4 = stat[col];
            lse = s4.x, mu = s4.y, eps = s4.z, sub = s4.w;
            i = l0 + 16 * piece + col;
            j = own_idx;
          } else {
            lse = r_lse, mu = r_mu, eps = r_eps, sub = r_sub;
            i = own_idx;
            j = l0 + 16 * piece + col;
          }
          float arg = fmaf(__uint_as_float(s[col]), scale_log2, -lse);
          if constexpr (MK == 2) arg = fmaf(unpack1<T>(mraw[col]), kLog2e, arg);  // scores are in log2 units
          float p = fast_exp2(arg);
          if constexpr (BOOLM)
            if (mraw[col] == 0u) p = 0.f;
          if (partial && (j >= n_valid || (causal && j > i))) p = 0.f;
          pv[h] = p;
          if constexpr (HAS_GT) {
            const float tm = fmaf(__uint_as_float(ts[col]), a.sm_scale, -mu);
            const float eb = __uint_as_float(e[col]) - eps;
            av[h] = p * tm;
            gt[h] = p * eb;
            gs[h] = p * fmaf(eb, tm, __uint_as_float(fp[col]) - sub);
          } else {
            gs[h] = p * (__uint_as_float(fp[col]) - sub);
          }
        }
        pk_gs[x2] = Elem<T>::pack(gs[0], gs[1]);
        if constexpr (HAS_GT) pk_gt[x2] = Elem<T>::pack(gt[0], gt[1]);
        if constexpr (HAS_GT && OWN_KEYS) pk_av[x2] = Elem<T>::pack(av[0], av[1]);
        if constexpr (OWN_KEYS) pk_p[x2] = Elem<T>::pack(pv[0], pv[1]);
      }
      // over this thread's own 16 columns of S and TS, all of which are in registers
      tmem_st8(sc + C::COL_S, pk_gs);
      if constexpr (HAS_GT) tmem_st8(sc + C::COL_S + 8, pk_gt);
      if constexpr (HAS_GT && OWN_KEYS) tmem_st8(sc + C::COL_TS, pk_av);
      if constexpr (OWN_KEYS && (HAS_GO || !HAS_GT)) tmem_st8(sc + C::COL_TS + 8, pk_p);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(p_full + (t & 1));
    }

    // ---- epilogue ----
    if (alive && n_tiles > 0) alive = mbar_wait(done, 0, ab, kAbortBwdDone);
    if (alive) {
      tc_fence_after();
      const bool in_range = own_idx < L;
      auto store_rows = [&](void* gptr, uint32_t col0, float mul) {
        T* g = reinterpret_cast<T*>(gptr) + ((size_t)bh * L + own_idx) * D;
        for (int c = piece; c < D / 32; c += NP) {  // 32-column chunks dealt round the warpgroups
          uint32_t r[32], pk[16];
          if (n_tiles > 0) {
            tmem_ld32(tbase + col0 + 32 * c, r);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int x = 0; x < 32; ++x) r[x] = 0u;
          }
#pragma unroll
          for (int x = 0; x < 16; ++x)
            pk[x] = Elem<T>::pack(__uint_as_float(r[2 * x]) * mul, __uint_as_float(r[2 * x + 1]) * mul);
          if (in_range) {
#pragma unroll
            for (int x = 0; x < 4; ++x)
              reinterpret_cast<uint4*>(g + 32 * c)[x] = make_uint4(pk[4 * x], pk[4 * x + 1], pk[4 * x + 2], pk[4 * x + 3]);
          }
        }
      };
      if constexpr (OWN_KEYS) {
        store_rows(a.dk, C::COL_OUT0, a.sm_scale);
        store_rows(a.dv, C::COL_OUT1, 1.f);
      } else {
        store_rows(a.dq, C::COL_OUT0, a.sm_scale);
      }
    }
  }

  // The own-queries launch may have started while the own-keys launch before it was still running (programmatic
  // stream serialization).  Whatever follows on the stream is ordered after THIS grid only, so this grid must not
  // complete before that one has: wait for it here, after the work.
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
template <typename T, bool OWN_KEYS, bool HAS_GO, bool HAS_GT, int MK>
static int launch_pipe_half(const jvpfa_bwd_args& a, cudaStream_t stream, int* status, bool overlap_previous) {
  using C = BwdPipeCfg<OWN_KEYS, HAS_GO, HAS_GT>;
  BwdPipeMaps m;
  const CUtensorMapDataType dt = Fmt<T>::kTma;
  const int key_rows = OWN_KEYS ? C::OWN : C::BL;
  const int qry_rows = OWN_KEYS ? C::BL : C::OWN;
  auto enc = [&](CUtensorMap* map, const void* p, const int64_t* st, int rows) {
    return encode_map4d(map, dt, p, C::D, a.L, a.H, a.B, st, rows);
  };
  bool ok = enc(&m.k, a.k, a.in_stride, key_rows) && enc(&m.v, a.v, a.in_stride, key_rows) &&
            enc(&m.q, a.q, a.in_stride, qry_rows);
  m.tk = m.tv = m.k;
  m.go = m.tq = m.g = m.q;
  if (HAS_GO) ok = ok && enc(&m.go, a.go, nullptr, qry_rows);
  if (HAS_GT)
    ok = ok && enc(&m.tk, a.tk, a.in_stride, key_rows) && enc(&m.tv, a.tv, a.in_stride, key_rows) &&
         enc(&m.tq, a.tq, a.in_stride, qry_rows) && enc(&m.g, a.gto, nullptr, qry_rows);
  if (!ok) {
    set_last_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled(bwd)");
    return JVPFA_ERR_CUDA;
  }
  auto kern = bwd_tc5_pipe128_kernel<T, OWN_KEYS, HAS_GO, HAS_GT, MK>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
  if (e != cudaSuccess) {
    set_last_cuda_error(e, "cudaFuncSetAttribute(bwd_tc5_pipe128)");
    return JVPFA_ERR_CUDA;
  }
  dim3 grid((a.L + C::OWN - 1) / C::OWN, a.B * a.H);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid, cfg.blockDim = dim3(C::NTHREADS);
  cfg.dynamicSmemBytes = C::SMEM_BYTES, cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = overlap_previous ? 1 : 0;
  e = cudaLaunchKernelEx(&cfg, kern, a, m, status);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_cuda_error(e, "launch bwd_tc5_pipe128");
    return JVPFA_ERR_CUDA;
  }
  return JVPFA_OK;
}

template <typename T, bool HAS_GO, bool HAS_GT, int MK>
static int launch_pipe_both(const jvpfa_bwd_args& a, cudaStream_t s) {
  int* status = tc5_status_device_ptr();
  if (!status) {
    set_last_cuda_error(cudaErrorUnknown, "status word address");
    return JVPFA_ERR_CUDA;
  }
  int rc = launch_pipe_half<T, true, HAS_GO, HAS_GT, MK>(a, s, status, false);
  if (rc) return rc;
  return launch_pipe_half<T, false, HAS_GO, HAS_GT, MK>(a, s, status, true);
}

template <typename T, int MK>
static int launch_pipe_m(const jvpfa_bwd_args& a, cudaStream_t s) {
  const bool go = a.go != nullptr, gt = a.gto != nullptr;
  if (go && gt) return launch_pipe_both<T, true, true, MK>(a, s);
  if (gt) return launch_pipe_both<T, false, true, MK>(a, s);
  return launch_pipe_both<T, true, false, MK>(a, s);
}

template <typename T>
static int launch_pipe_t(const jvpfa_bwd_args& a, cudaStream_t s) {
  if (a.mask.kind == JVPFA_MASK_BOOL && a.mask_tile_live != nullptr && a.mask_tile_live_t != nullptr)
    return launch_pipe_m<T, 3>(a, s);
  if (a.mask.kind == JVPFA_MASK_BOOL) return launch_pipe_m<T, 1>(a, s);
  if (a.mask.kind == JVPFA_MASK_BIAS) return launch_pipe_m<T, 2>(a, s);
  return launch_pipe_m<T, 0>(a, s);
}

}  // namespace tc5

// Every request that bwd_tc5_eligible() accepts with head dimension 128 (it checks the mask layout).
bool bwd_tc5_pipe128_eligible(const jvpfa_bwd_args& a) {
  return (a.dtype == JVPFA_BF16 || a.dtype == JVPFA_FP16) && a.D == 128;
}

int launch_bwd_tc5_pipe128(const jvpfa_bwd_args& a, cudaStream_t s) {
  return a.dtype == JVPFA_BF16 ? tc5::launch_pipe_t<__nv_bfloat16>(a, s) : tc5::launch_pipe_t<__half>(a, s);
}

}  // namespace jvpfa
