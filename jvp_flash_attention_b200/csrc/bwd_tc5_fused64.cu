// Single-pass tcgen05 backward for head dimension 64 (bf16 / fp16; none, causal, key padding): the score
// tiles S, tS, E, FP are formed ONCE per (128 keys x 64 queries) sub-tile and feed all three gradients.
//
// The two-launch backward (bwd_tc5_d64.cu, like upstream's _attn_bwd_dkdv / _attn_bwd_dq,
// jvp_attention.py:1415-1707) recomputes the score tiles in the launch that owns queries: 15 MMAs are
// executed for 10 needed.  Here one persistent CTA per SM owns 128 keys (keys <-> TMEM lanes), streams the
// queries in sub-tiles of 64 and produces
//     dK += gS^T Q + gtS^T tQ,   dV += A^T G (+ P^T gO)            accumulated in TMEM over the sub-tiles,
//     dQ[sub-tile] = gS K + gtS tK                                 one 64 x 64 product per sub-tile,
// The dQ product contracts over the keys, i.e. over TMEM lanes, so its operands cannot come from TMEM: the
// elementwise threads write gS and gtS as 16-bit tiles [key][query] into SHARED memory.  That one layout is a
// K-major A operand for the dK products (M = keys) and an MN-major A operand for the dQ product (M = 64
// queries, K = keys); K / tK are its MN-major B operand.  A and P, which only dV needs, stay in TMEM.  Handing the operands over through
// shared memory also frees the score accumulators as soon as the elementwise threads hold them in
// registers, so the scores of sub-tile g+1 are formed while sub-tile g is still being worked on.
// A dQ sub-tile is read back by a fourth warpgroup (an M = 64 accumulator sits in lanes 0..15 of each
// 32-lane quarter) and added to an fp32 accumulation buffer in global memory with vector reductions
// (red.global.add.v4.f32); a small kernel converts that buffer to the output type at the end.  The order of
// those additions varies from run to run, so dQ is reproducible to rounding, not bitwise.
//
// Warps: 0 TMA producer (+ per-query statistics), 1 score issuer, 2 dK/dV issuer, 3 dQ issuer,
// 4..11 two elementwise warpgroups (thread <-> key row; group w takes query columns [32w, 32w+32) of every
// sub-tile), 12..15 dQ read-back.  (Four elementwise warpgroups of 16 columns each, taking turns at the
// read-back, were measured slower: 0.284 ms against 0.261 ms on the B4 H16 L2048 causal shape.)
// TMEM (512 columns): S | tS | E | FP (64 each) ; dK | dV (64 each) ; dQ (64) ; packed A | P (32 each).
#include "tc5_common.cuh"

namespace jvpfa {
namespace tc5 {

struct BwdFMaps {
  CUtensorMap k, v, tk, tv;  // key side, box 128 rows
  CUtensorMap q, go, tq, g;  // query side, box 64 rows (g = cotangent of tO)
  CUtensorMap dq;            // the fp32 dQ accumulation buffer, box 64 rows x 32 columns
};

// TMA reduction (add) of one fp32 tile from shared memory into global memory; rows past the tensor's extent are
// not touched.
__device__ __forceinline__ void tma_reduce_add_4d(const CUtensorMap* map, uint32_t smem_src, int x, int y, int z, int w) {
  asm volatile("cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(map),
               "r"(smem_src), "r"(x), "r"(y), "r"(z), "r"(w)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

template <bool HAS_GO, bool HAS_GT>
struct BwdFCfg {
  static constexpr int D = 64;
  static constexpr int OWN = 128;
  static constexpr int BL = 64;
  static constexpr int STAGES = (HAS_GO && HAS_GT) ? 2 : 3;
  // The shared-memory result tiles (gS, gtS) exist twice, so that the elementwise threads can write sub-tile g + 1
  // while the products of sub-tile g still read theirs.
  static constexpr int N_OBUF = 2;
  static constexpr int NTHREADS = 512;
  static constexpr int N_OWN = HAS_GT ? 4 : 2;                           // K, tK, V, tV | K, V
  static constexpr int N_LOOP = 1 + (HAS_GO ? 1 : 0) + (HAS_GT ? 2 : 0);  // Q, tQ, G, gO
  static constexpr int N_OUT = 1 + (HAS_GT ? 1 : 0);                      // gS, gtS (A and P stay in TMEM)
  static constexpr int OWN_BYTES = OWN * D * 2;   // 16 KiB
  static constexpr int LOOP_BYTES = BL * D * 2;   // 8 KiB
  static constexpr int OUT_BYTES = OWN * BL * 2;  // 16 KiB: [128 keys][64 queries]
  static constexpr int STAGE_BYTES = N_LOOP * LOOP_BYTES;
  static constexpr int STAT_STAGE_BYTES = (BL / 2) * 32;  // per query pair two float4
  // Two sets of own tiles where shared memory allows it (backward through O alone: K and V only): the next item's
  // are then loaded while this item's last sub-tiles run.  With one set the item boundary is exposed - the next
  // load can only be requested when the last dQ product has completed (about an eighth of the kernel's time).
  static constexpr int OWN_BUFS = HAS_GT ? 1 : 2;
  static constexpr int OWN_SET_BYTES = N_OWN * OWN_BYTES;
  static constexpr int OFF_OWN = 0;
  static constexpr int OFF_RING = OWN_BUFS * OWN_SET_BYTES;
  static constexpr int OFF_OUT = OFF_RING + STAGES * STAGE_BYTES;
  static constexpr int OBUF_BYTES = N_OUT * OUT_BYTES;
  static constexpr int OFF_STAT = OFF_OUT + N_OBUF * OBUF_BYTES;
  // dQ of a sub-tile on its way out: fp32 [64 queries][64 columns] as two 128-byte-swizzled halves of 32 columns
  static constexpr int OFF_DQS = OFF_STAT + STAGES * STAT_STAGE_BYTES;
  static constexpr int DQS_BYTES = BL * D * 4;
  static_assert(OFF_DQS % 1024 == 0, "swizzled staging tile alignment");
  static constexpr int TILE_BYTES = OFF_DQS + DQS_BYTES;
  static constexpr int SMEM_NEEDED = TILE_BYTES + 512 + 1024;
  // At least 120 KiB so that a second CTA can never share the SM (the CTA allocates all of TMEM).
  static constexpr int SMEM_BYTES = SMEM_NEEDED > 120 * 1024 ? SMEM_NEEDED : 120 * 1024;
  static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
  static constexpr int SLOT_K = 0, SLOT_TK = 1, SLOT_V = HAS_GT ? 2 : 1, SLOT_TV = 3;
  static constexpr int SLOT_Q = 0, SLOT_TQ = 1, SLOT_G = 2, SLOT_GO = HAS_GT ? 3 : 1;
  static constexpr int OUT_GS = 0, OUT_GT = 1;
  static constexpr int COL_S = 0, COL_TS = 64, COL_E = 128, COL_FP = HAS_GT ? 192 : 64;
  static constexpr int COL_DK = 256, COL_DV = 320, COL_DQ = 384;
  static constexpr int COL_AV = 448, COL_P = 480;  // packed 16-bit A and P: TMEM operands of the dV products
  static constexpr int COLS_ALLOC = 512;
};

__device__ __forceinline__ float2 ff(uint32_t a, uint32_t b) { return make_float2(__uint_as_float(a), __uint_as_float(b)); }
__device__ __forceinline__ void sts_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]; descriptor low words as in umma_ss_lo, accumulate flag known at run time.
__device__ __forceinline__ void mma_ss_dyn(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(kDescHi), "r"(idesc), "r"(accumulate)
      : "memory");
}

struct FItem {
  int bh, b, h, own0, loop_begin, n_sub;
};

// MK: 0 = none / causal / key padding (index comparisons); 1 = uint8 mask with any strides (each elementwise thread
// reads the 32 mask bytes of its key row and the sub-tile's queries before it waits for the scores); 2 = additive bias of
// the element type, read the same way (HAS_GT == false only).
template <typename T, bool HAS_GO, bool HAS_GT, int MK>
__global__ void __launch_bounds__(512, 1)
bwd_tc5_fused64_kernel(const jvpfa_bwd_args a, const __grid_constant__ BwdFMaps maps, float* dq_acc, int* status) {
  using C = BwdFCfg<HAS_GO, HAS_GT>;
  constexpr int D = 64, OWN = C::OWN, BL = C::BL, STAGES = C::STAGES;

  const bool dead_on_entry = *(volatile int*)status != 0;  // an earlier bounded wait gave up

  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  unsigned char* smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  unsigned char* sOwn = smem + C::OFF_OWN;
  unsigned char* sRing = smem + C::OFF_RING;
  unsigned char* sOut = smem + C::OFF_OUT;
  float4* sStat = reinterpret_cast<float4*>(smem + C::OFF_STAT);  // [STAGES][BL/2][2]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::TILE_BYTES);
  uint64_t* own_full = bars + 0;             // [2] per set of own tiles (item kact uses set kact % OWN_BUFS)
  uint64_t* own_free = bars + 2;             // [2] score issuer + dQ issuer are through with the set
  uint64_t* loop_full = bars + 4;            // [STAGES]
  uint64_t* loop_empty = loop_full + STAGES;  // [STAGES]: score issuer + dK/dV issuer
  uint64_t* stat_full = loop_empty + STAGES;  // [STAGES]
  uint64_t* s_full = stat_full + STAGES;
  uint64_t* s_free = s_full + 1;    // 256 elementwise threads hold the scores in registers
  // [2] by g & 1, 256 each: gS, gtS, A, P of the sub-tile are in shared memory. A pair, because the elementwise
  // threads can finish sub-tile g + 1 before the dQ issuer has looked at g (sub-tile g + 1 needs the dV products of
  // g, not its dQ product): on one barrier the issuer would then be two phases behind, where a parity wait no longer
  // tells "done" from "not yet". Sub-tile g + 2 does need dQ of g (out_free), so one phase per barrier is the most.
  uint64_t* p_full = s_free + 1;
  uint64_t* out_free = p_full + 2;  // [2] per result buffer: dK/dV issuer + dQ issuer have read it
  uint64_t* av_free = out_free + 2;  // the dV products have read the packed A / P columns
  uint64_t* dq_full = av_free + 1;
  uint64_t* dq_free = dq_full + 1;   // 128 read-back threads
  uint64_t* done = dq_free + 1;      // the item's dK / dV are complete
  uint64_t* acc_free = done + 1;     // 256: the epilogue has read them
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_free + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* rb_ok = reinterpret_cast<volatile int*>(tmem_slot + 2);  // the read-back group's poller tells the rest

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int L = a.L;
  const int BH = a.B * a.H;
  const bool causal = a.mask.kind == JVPFA_MASK_CAUSAL;
  const int n_own_tiles = (L + OWN - 1) / OWN;
  const int n_items = n_own_tiles * BH;
  const int G = (int)gridDim.x, cta = (int)blockIdx.x;
  const int k_max = (n_items + G - 1) / G;

  // Item k of this CTA: ranked heaviest first (causal: the first key tile sees every query), dealt in serpentine order.
  auto get_item = [&](int k, FItem& it) -> bool {
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
    it.own0 = rank * OWN;
    it.loop_begin = causal ? (it.own0 / BL) * BL : 0;
    it.n_sub = (L - it.loop_begin + BL - 1) / BL;
    if (it.own0 >= n_valid) it.n_sub = 0;
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

  // NaN into the rows of dK, dV and of the dQ accumulator that this CTA's items own: this launch's results are
  // not to be trusted
  auto poison = [&]() {
    FItem it;
    for (int k = 0; k < k_max; ++k) {
      if (!get_item(k, it)) continue;
      const int i = it.own0 + tid;
      if (tid < OWN && i < L) {
        poison_row<T>(a.dk, (size_t)it.bh * L + i, D);
        poison_row<T>(a.dv, (size_t)it.bh * L + i, D);
        dq_acc[((size_t)it.bh * L + i) * D] = poison_f32();
      }
    }
  };
  if (dead_on_entry) {
    poison();
    return;
  }

  if (tid == 0) {
    mbar_init(own_full, 1);
    mbar_init(own_full + 1, 1);
    mbar_init(own_free, 2);
    mbar_init(own_free + 1, 2);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(loop_full + s, 1);
      mbar_init(loop_empty + s, 2);
      mbar_init(stat_full + s, 1);
    }
    mbar_init(s_full, 1);
    mbar_init(s_free, 256);
    mbar_init(p_full, 256);
    mbar_init(p_full + 1, 256);
    mbar_init(out_free, 2);
    mbar_init(out_free + 1, 2);
    mbar_init(av_free, 1);
    mbar_init(dq_full, 1);
    mbar_init(dq_free, 128);
    mbar_init(done, 1);
    mbar_init(acc_free, 256);
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

  // Registers: the elementwise threads hold four 32-column accumulator slices; everybody else needs few.
  // (setmaxnreg.inc draws on what setmaxnreg.dec of the same CTA has released and blocks until it is there: 256
  // threads x 56 registers up equals 256 threads x 56 registers down from the 128 the kernel is launched with.)
  if (warp < 4 || warp >= 12) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 184;");
  }

  // Phase counters kept alike by all roles: g counts the sub-tiles of this CTA (ring stage g % STAGES, dQ buffer
  // g & 1; s_full, s_free complete once per sub-tile, p_full and out_free of buffer g & 1 every other one), kact the items that have sub-tiles.
  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer + per-query statistics
    if (lane == 0) {
      prefetch_tmap(&maps.k), prefetch_tmap(&maps.v), prefetch_tmap(&maps.q);
      if constexpr (HAS_GO) prefetch_tmap(&maps.go);
      if constexpr (HAS_GT) prefetch_tmap(&maps.tk), prefetch_tmap(&maps.tv), prefetch_tmap(&maps.tq), prefetch_tmap(&maps.g);
    }
    struct Stat {
      float lse[2], delta[2], mu[2], eps[2], cterm[2];
    };
    int g = 0, kact = 0;
    bool ok = true;
    FItem it;
    for (int k = 0; ok && k < k_max; ++k) {
      if (!get_item(k, it) || it.n_sub == 0) continue;
      // The own tiles are single-buffered: every MMA that reads the previous item's must be complete.
      const int oset = kact % C::OWN_BUFS, ouse = kact / C::OWN_BUFS;  // set of own tiles and how often it was used
      if (ouse > 0 && !mbar_wait_backoff(own_free + oset, (ouse - 1) & 1, ab, kAbortBwdOwn)) break;
      if (lane == 0) {
        unsigned char* dst = sOwn + oset * C::OWN_SET_BYTES;
        uint64_t* full = own_full + oset;
        mbar_expect_tx(full, C::N_OWN * C::OWN_BYTES);
        tma_load_4d(dst + C::SLOT_K * C::OWN_BYTES, &maps.k, full, 0, it.own0, it.h, it.b);
        tma_load_4d(dst + C::SLOT_V * C::OWN_BYTES, &maps.v, full, 0, it.own0, it.h, it.b);
        if constexpr (HAS_GT) {
          tma_load_4d(dst + C::SLOT_TK * C::OWN_BYTES, &maps.tk, full, 0, it.own0, it.h, it.b);
          tma_load_4d(dst + C::SLOT_TV * C::OWN_BYTES, &maps.tv, full, 0, it.own0, it.h, it.b);
        }
      }
      const size_t stat_off = (size_t)it.bh * L;
      // lane l holds the statistics of queries 2l, 2l+1 of a sub-tile; fetched one sub-tile ahead of their use
      auto load_stats = [&](int s, Stat& r) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          r.lse[e] = INFINITY, r.delta[e] = r.mu[e] = r.eps[e] = r.cterm[e] = 0.f;
          const int i = it.loop_begin + s * BL + 2 * lane + e;
          if (s < it.n_sub && i < L) {
            r.lse[e] = a.lse[stat_off + i];
            r.delta[e] = a.delta[stat_off + i];
            if constexpr (HAS_GT) {
              r.mu[e] = a.mu[stat_off + i];
              r.eps[e] = a.eps[stat_off + i];
              r.cterm[e] = a.cterm[stat_off + i];
            }
          }
        }
      };
      Stat cur, nxt;
      load_stats(0, cur);
      for (int s = 0; s < it.n_sub; ++s, ++g) {
        const int st = g % STAGES;
        if (!mbar_wait_backoff(loop_empty + st, ((g / STAGES) & 1) ^ 1, ab, kAbortBwdLoopEmpty)) {
          ok = false;
          break;
        }
        const int l0 = it.loop_begin + s * BL;
        if (lane == 0) {
          unsigned char* base = sRing + st * C::STAGE_BYTES;
          mbar_expect_tx(loop_full + st, C::STAGE_BYTES);
          tma_load_4d(base + C::SLOT_Q * C::LOOP_BYTES, &maps.q, loop_full + st, 0, l0, it.h, it.b);
          if constexpr (HAS_GO) tma_load_4d(base + C::SLOT_GO * C::LOOP_BYTES, &maps.go, loop_full + st, 0, l0, it.h, it.b);
          if constexpr (HAS_GT) {
            tma_load_4d(base + C::SLOT_TQ * C::LOOP_BYTES, &maps.tq, loop_full + st, 0, l0, it.h, it.b);
            tma_load_4d(base + C::SLOT_G * C::LOOP_BYTES, &maps.g, loop_full + st, 0, l0, it.h, it.b);
          }
        }
        load_stats(s + 1, nxt);
        // negated and stored pairwise for the packed arithmetic:
        //   float4 A = (-lse0, -lse1, -mu0, -mu1), float4 B = (-eps0, -eps1, -sub0, -sub1)
        float4* dst = sStat + (st * (BL / 2) + lane) * 2;
        dst[0] = make_float4(-cur.lse[0], -cur.lse[1], -cur.mu[0], -cur.mu[1]);
        dst[1] = make_float4(-cur.eps[0], -cur.eps[1], -(cur.delta[0] + cur.cterm[0] + cur.eps[0] * cur.mu[0]),
                             -(cur.delta[1] + cur.cterm[1] + cur.eps[1] * cur.mu[1]));
        __syncwarp();
        if (lane == 0) mbar_arrive(stat_full + st);
        cur = nxt;
      }
      ++kact;
    }
  } else if (warp <= 3) {
    if (lane == 0) {
      constexpr uint32_t idesc_sc = make_idesc(Fmt<T>::kIdesc, OWN, BL, 0, 0);       // 128 x 64 scores
      constexpr uint32_t idesc_sc2 = make_idesc(Fmt<T>::kIdesc, OWN, 2 * BL, 0, 0);  // 128 x 128: [S | tS]
      constexpr uint32_t idesc_kv = make_idesc(Fmt<T>::kIdesc, OWN, D, 0, 1);        // dK, dV: 128 x 64, B MN-major
      constexpr uint32_t idesc_dq = make_idesc(Fmt<T>::kIdesc, BL, D, 1, 1);         // dQ: 64 x 64, A and B MN-major
      // MN-major operands made of one 64-element chunk: the leading offset is not used (any value), 8-row groups 1024 B
      constexpr uint32_t kLoMN = (uint32_t)(8192 >> 4) << 16;
      constexpr uint32_t OWN16 = C::OWN_BYTES >> 4, LOOP16 = C::LOOP_BYTES >> 4, OUT16 = C::OUT_BYTES >> 4,
                         STAGE16 = C::STAGE_BYTES >> 4;
      const uint32_t own_k0 = kDescLo | (smem_u32(sOwn) >> 4);    // own tiles (first set) as K-major A operands
      const uint32_t own_mn0 = kLoMN | (smem_u32(sOwn) >> 4);     // ... as MN-major B operands (dQ)
      constexpr uint32_t OWNSET16 = C::OWN_SET_BYTES >> 4;
      const uint32_t ring_k = kDescLo | (smem_u32(sRing) >> 4);  // streamed tiles as K-major B operands (scores)
      const uint32_t ring_mn = kLoMN | (smem_u32(sRing) >> 4);   // ... as MN-major B operands (dK, dV)
      const uint32_t out_k = kDescLo | (smem_u32(sOut) >> 4);    // elementwise results as K-major A operands (dK, dV)
      const uint32_t out_mn = kLoMN | (smem_u32(sOut) >> 4);     // ... as MN-major A operands (dQ)
      int g = 0, kact = 0;
      bool ok = true;
      FItem it;
      if (warp == 1) {
        // ---------------------------------------------------------------- scores
        uint32_t own_k = own_k0;  // this item's set
        auto score = [&](uint32_t col, uint32_t own_slot, uint32_t b_lo, uint32_t id, bool first) {
          const uint32_t a_lo = own_k + own_slot * OWN16;
          if (first)
            umma_ss_lo<false>(tmem + col, a_lo, b_lo, id);
          else
            umma_ss_lo<true>(tmem + col, a_lo, b_lo, id);
#pragma unroll
          for (int ks = 1; ks < D / 16; ++ks) umma_ss_lo<true>(tmem + col, a_lo + ks * 2, b_lo + ks * 2, id);
        };
        for (int k = 0; ok && k < k_max; ++k) {
          if (!get_item(k, it) || it.n_sub == 0) continue;
          const int oset = kact % C::OWN_BUFS;
          if (!mbar_wait(own_full + oset, (kact / C::OWN_BUFS) & 1, ab, kAbortBwdOwn)) break;
          own_k = own_k0 + oset * OWNSET16;
          for (int s = 0; s < it.n_sub; ++s, ++g) {
            const int st = g % STAGES;
            if (!mbar_wait(loop_full + st, (g / STAGES) & 1, ab, kAbortBwdLoopFull) ||
                (g > 0 && !mbar_wait(s_free, (g - 1) & 1, ab, kAbortBwdSFull))) {
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t lp = ring_k + st * STAGE16;
            if constexpr (HAS_GT) {
              score(C::COL_S, C::SLOT_K, lp + C::SLOT_Q * LOOP16, idesc_sc2, true);    // [S | tS] = K [Q ; tQ]^T
              score(C::COL_TS, C::SLOT_TK, lp + C::SLOT_Q * LOOP16, idesc_sc, false);  // tS += tK Q^T
              score(C::COL_E, C::SLOT_V, lp + C::SLOT_G * LOOP16, idesc_sc, true);     // E = V G^T
              score(C::COL_FP, C::SLOT_TV, lp + C::SLOT_G * LOOP16, idesc_sc, true);   // FP = tV G^T
              if constexpr (HAS_GO) score(C::COL_FP, C::SLOT_V, lp + C::SLOT_GO * LOOP16, idesc_sc, false);  // + V gO^T
            } else {
              score(C::COL_S, C::SLOT_K, lp + C::SLOT_Q * LOOP16, idesc_sc, true);    // S = K Q^T
              score(C::COL_FP, C::SLOT_V, lp + C::SLOT_GO * LOOP16, idesc_sc, true);  // FP = V gO^T
            }
            tc_commit(s_full);
            tc_commit(loop_empty + st);
          }
          if (!ok) break;
          tc_commit(own_free + oset);
          ++kact;
        }
      } else if (warp == 2) {
        // ---------------------------------------------------------------- dK, dV
        // out (+)= result tile (A, K-major: 128 keys x 64 queries) x streamed tile (B, MN-major: 64 queries x 64)
        uint32_t ob16 = 0;  // result buffer of the sub-tile, in 16-byte units
        auto outer = [&](uint32_t col, uint32_t out_slot, uint32_t b_lo, uint32_t accumulate) {
          const uint32_t a_lo = out_k + ob16 + out_slot * OUT16;
          mma_ss_dyn(tmem + col, a_lo, b_lo, idesc_kv, accumulate);
#pragma unroll
          for (int ks = 1; ks < BL / 16; ++ks) umma_ss_lo<true>(tmem + col, a_lo + ks * 2, b_lo + ks * 128, idesc_kv);
        };
        // out (+)= packed operand (A, TMEM: 8 columns per 16 queries) x streamed tile (B, MN-major)
        auto outer_t = [&](uint32_t col, uint32_t a_col, uint32_t b_lo, uint32_t accumulate) {
          umma_ts_lo_dyn(tmem + col, tmem + a_col, b_lo, idesc_kv, accumulate);
#pragma unroll
          for (int ks = 1; ks < BL / 16; ++ks) umma_ts_lo<true>(tmem + col, tmem + a_col + ks * 8, b_lo + ks * 128, idesc_kv);
        };
        for (int k = 0; ok && k < k_max; ++k) {
          if (!get_item(k, it) || it.n_sub == 0) continue;
          for (int s = 0; s < it.n_sub; ++s, ++g) {
            const int st = g % STAGES;
            if (!mbar_wait(p_full + (g & 1), (g >> 1) & 1, ab, kAbortBwdPFull) ||
                (s == 0 && kact > 0 && !mbar_wait(acc_free, (kact - 1) & 1, ab, kAbortBwdDone))) {
              ok = false;
              break;
            }
            tc_fence_after();
            const int ob = g % C::N_OBUF;
            ob16 = ob * (C::OBUF_BYTES >> 4);
            const uint32_t lp = ring_mn + st * STAGE16;
            const uint32_t acc = s > 0;
            outer(C::COL_DK, C::OUT_GS, lp + C::SLOT_Q * LOOP16, acc);  // dK += gS^T Q
            if constexpr (HAS_GT) {
              outer(C::COL_DK, C::OUT_GT, lp + C::SLOT_TQ * LOOP16, 1);  // dK += gtS^T tQ
              outer_t(C::COL_DV, C::COL_AV, lp + C::SLOT_G * LOOP16, acc);  // dV += A^T G
              if constexpr (HAS_GO) outer_t(C::COL_DV, C::COL_P, lp + C::SLOT_GO * LOOP16, 1);  // dV += P^T gO
            } else {
              outer_t(C::COL_DV, C::COL_P, lp + C::SLOT_GO * LOOP16, acc);  // dV += P^T gO
            }
            tc_commit(loop_empty + st);
            tc_commit(out_free + ob);
            tc_commit(av_free);
          }
          if (!ok) break;
          tc_commit(done);
          ++kact;
        }
      } else {
        // ---------------------------------------------------------------- dQ of the sub-tile
        // dQ (+)= result tile (A, MN-major: 64 queries x 128 keys) x own tile (B, MN-major: 128 keys x 64)
        uint32_t ob16 = 0;
        uint32_t own_mn = own_mn0;  // this item's set
        auto inner = [&](uint32_t col, uint32_t out_slot, uint32_t own_slot, bool first) {
          const uint32_t a_lo = out_mn + ob16 + out_slot * OUT16, b_lo = own_mn + own_slot * OWN16;
          if (first)
            umma_ss_lo<false>(tmem + col, a_lo, b_lo, idesc_dq);
          else
            umma_ss_lo<true>(tmem + col, a_lo, b_lo, idesc_dq);
#pragma unroll
          for (int ks = 1; ks < OWN / 16; ++ks) umma_ss_lo<true>(tmem + col, a_lo + ks * 128, b_lo + ks * 128, idesc_dq);
        };
        for (int k = 0; ok && k < k_max; ++k) {
          if (!get_item(k, it) || it.n_sub == 0) continue;
          own_mn = own_mn0 + (kact % C::OWN_BUFS) * OWNSET16;
          for (int s = 0; s < it.n_sub; ++s, ++g) {
            if (!mbar_wait(p_full + (g & 1), (g >> 1) & 1, ab, kAbortBwdPFull) ||
                (g >= 1 && !mbar_wait(dq_free, (g - 1) & 1, ab, kAbortBwdDone))) {
              ok = false;
              break;
            }
            tc_fence_after();
            const int ob = g % C::N_OBUF;
            ob16 = ob * (C::OBUF_BYTES >> 4);
            const uint32_t col = C::COL_DQ;
            inner(col, C::OUT_GS, C::SLOT_K, true);                       // dQ = gS K
            if constexpr (HAS_GT) inner(col, C::OUT_GT, C::SLOT_TK, false);  // dQ += gtS tK
            tc_commit(dq_full);
            tc_commit(out_free + ob);
          }
          if (!ok) break;
          tc_commit(own_free + kact % C::OWN_BUFS);
          ++kact;
        }
      }
    }
  } else if (warp < 12) {
    // ------------------------------------------------------------------ elementwise warpgroups
    const int wg = (warp - 4) >> 2;  // 0 / 1: query columns [32 wg, 32 wg + 32) of every sub-tile
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;  // key row of the own tile <-> TMEM lane
    const uint32_t tbase = tmem + ((uint32_t)(quarter * 32) << 16) + 32 * wg;
    const float2 c2 = make_float2(a.sm_scale * kLog2e, a.sm_scale * kLog2e);
    const float2 sc2 = make_float2(a.sm_scale, a.sm_scale);
    // this thread's row of the result tiles: 16-byte chunk c (8 queries) sits at position c ^ (row & 7)
    const uint32_t out_row = smem_u32(sOut) + row * 128;
    const uint32_t sw = (uint32_t)(row & 7);
    bool alive = true;
    int g = 0, kact = 0;
    FItem it;

    auto store_row = [&](void* gptr, int bh, int own_idx, const uint32_t (&r0)[32], const uint32_t (&r1)[32], float mul) {
      if (own_idx >= L) return;
      T* gp = reinterpret_cast<T*>(gptr) + ((size_t)bh * L + own_idx) * D;
#pragma unroll
      for (int x = 0; x < 4; ++x)
        reinterpret_cast<uint4*>(gp)[x] = make_uint4(
            Elem<T>::pack(__uint_as_float(r0[8 * x]) * mul, __uint_as_float(r0[8 * x + 1]) * mul),
            Elem<T>::pack(__uint_as_float(r0[8 * x + 2]) * mul, __uint_as_float(r0[8 * x + 3]) * mul),
            Elem<T>::pack(__uint_as_float(r0[8 * x + 4]) * mul, __uint_as_float(r0[8 * x + 5]) * mul),
            Elem<T>::pack(__uint_as_float(r0[8 * x + 6]) * mul, __uint_as_float(r0[8 * x + 7]) * mul));
#pragma unroll
      for (int x = 0; x < 4; ++x)
        reinterpret_cast<uint4*>(gp)[4 + x] = make_uint4(
            Elem<T>::pack(__uint_as_float(r1[8 * x]) * mul, __uint_as_float(r1[8 * x + 1]) * mul),
            Elem<T>::pack(__uint_as_float(r1[8 * x + 2]) * mul, __uint_as_float(r1[8 * x + 3]) * mul),
            Elem<T>::pack(__uint_as_float(r1[8 * x + 4]) * mul, __uint_as_float(r1[8 * x + 5]) * mul),
            Elem<T>::pack(__uint_as_float(r1[8 * x + 6]) * mul, __uint_as_float(r1[8 * x + 7]) * mul));
    };

    for (int k = 0; alive && k < k_max; ++k) {
      if (!get_item(k, it)) continue;
      const int own_idx = it.own0 + row;
      if (it.n_sub == 0) {
        // nothing attends these keys (they are all padding): the gradients are zero
        uint32_t z[32];
#pragma unroll
        for (int x = 0; x < 32; ++x) z[x] = 0u;
        store_row(wg == 0 ? a.dk : a.dv, it.bh, own_idx, z, z, 0.f);
        continue;
      }
      const int n_valid = valid_keys(it.b);
      for (int s = 0; s < it.n_sub; ++s, ++g) {
        const int st = g % STAGES;
        const int l0 = it.loop_begin + s * BL + 32 * wg;  // first query of this group's columns
        // MK = 1: this key's mask bytes for the 32 queries, requested before the waits (indices clamped into the
        // tensor; what lies outside is switched off by col_hi and by lse = +inf of the padding queries)
        // MK = 2 (backward through O alone: the variants with tangents have no registers to spare): the bias elements
        // of the same positions, 16 bit each, of the tensors' type.
        uint32_t mraw[MK != 0 ? 32 : 1];
        if constexpr (MK != 0) {
          constexpr int MESZ = MK == 1 ? 1 : 2;
          const unsigned char* pm = reinterpret_cast<const unsigned char*>(a.mask.ptr) +
                                    ((long long)it.b * a.mask.stride[0] + (long long)it.h * a.mask.stride[1] +
                                     (long long)min(own_idx, L - 1) * a.mask.stride[3]) * MESZ;
#pragma unroll
          for (int col = 0; col < 32; ++col) {
            const unsigned char* el = pm + (long long)min(l0 + col, L - 1) * a.mask.stride[2] * MESZ;
            mraw[col] = MK == 1 ? ldg_nc_u8(el) : ldg_nc_u16(el);
          }
        }
        if (!mbar_wait(stat_full + st, (g / STAGES) & 1, ab, kAbortBwdLoopFull) ||
            !mbar_wait(s_full, g & 1, ab, kAbortBwdSFull)) {
          alive = false;
          break;
        }
        tc_fence_after();
        uint32_t live = 0xffffffffu;  // MK = 1: bit col = the mask lets query l0 + col attend this key
        if constexpr (MK == 1) {
          live = 0u;
#pragma unroll
          for (int col = 0; col < 32; ++col) live |= (mraw[col] != 0u ? 1u : 0u) << col;
        }
        uint32_t sv[32], fp[32], ts[HAS_GT ? 32 : 1], ev[HAS_GT ? 32 : 1];
        tmem_ld32(tbase + C::COL_S, sv);
        tmem_ld32(tbase + C::COL_FP, fp);
        if constexpr (HAS_GT) {
          tmem_ld32(tbase + C::COL_TS, ts);
          tmem_ld32(tbase + C::COL_E, ev);
        }
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(s_free);
        // (key j = own_idx, query i = l0 + col) is dead if j >= n_valid, or causal and j > i: columns in [col_lo, col_hi) live
        int col_lo = 0, col_hi = 32;
        if (own_idx >= n_valid) col_hi = 0;
        if (causal) col_lo = own_idx - l0;
        const float4* stat = sStat + (st * (BL / 2) + 16 * wg) * 2;
        uint32_t pk_gs[16], pk_gt[HAS_GT ? 16 : 1], pk_av[HAS_GT ? 16 : 1], pk_p[HAS_GO ? 16 : 1];
        // One column pair: p from the scores and the row statistics, then the 16-bit operands.  MASKED: columns
        // outside [col_lo, col_hi) get p = 0.  Most sub-tiles have no dead pair for any thread of the warp and take
        // the variant without the comparisons and selects.
        auto pair = [&](int x, auto masked_c) {
          constexpr bool MASKED = decltype(masked_c)::value != 0;
          const int col = 2 * x;
          const float4 sa = stat[2 * x], sb = stat[2 * x + 1];
          const float2 nl = make_float2(sa.x, sa.y), nmu = make_float2(sa.z, sa.w);
          const float2 neps = make_float2(sb.x, sb.y), nsub = make_float2(sb.z, sb.w);
          float2 xs = __ffma2_rn(ff(sv[2 * x], sv[2 * x + 1]), c2, nl);
          if constexpr (MK == 2)  // scores are in log2 units: + bias * log2(e)
            xs = __ffma2_rn(unpack2<T>(mraw[2 * x] | (mraw[2 * x + 1] << 16)), make_float2(kLog2e, kLog2e), xs);
          float2 p = make_float2(fast_exp2(xs.x), fast_exp2(xs.y));
          if constexpr (MASKED) {
            if constexpr (MK == 1) {
              if (!((live >> col) & 1u)) p.x = 0.f;
              if (!((live >> (col + 1)) & 1u)) p.y = 0.f;
            } else {
              if (!(col >= col_lo && col < col_hi)) p.x = 0.f;
              if (!(col + 1 >= col_lo && col + 1 < col_hi)) p.y = 0.f;
            }
          }
          const float2 u = __fadd2_rn(ff(fp[2 * x], fp[2 * x + 1]), nsub);
          if constexpr (HAS_GT) {
            const float2 tm = __ffma2_rn(ff(ts[2 * x], ts[2 * x + 1]), sc2, nmu);
            const float2 eb = __fadd2_rn(ff(ev[2 * x], ev[2 * x + 1]), neps);
            const float2 av = __fmul2_rn(p, tm);
            const float2 gt = __fmul2_rn(p, eb);
            const float2 gs = __fmul2_rn(p, __ffma2_rn(eb, tm, u));
            pk_gs[x] = Elem<T>::pack(gs.x, gs.y);
            pk_gt[x] = Elem<T>::pack(gt.x, gt.y);
            pk_av[x] = Elem<T>::pack(av.x, av.y);
          } else {
            const float2 gs = __fmul2_rn(p, u);
            pk_gs[x] = Elem<T>::pack(gs.x, gs.y);
          }
          if constexpr (HAS_GO) pk_p[x] = Elem<T>::pack(p.x, p.y);
        };
        if constexpr (MK == 1) {  // the index range (key padding of the own tile) joins the mask bits
          const int lo = max(col_lo, 0), hi = min(col_hi, 32);
          live &= hi > lo ? ((hi - lo >= 32 ? 0xffffffffu : ((1u << (hi - lo)) - 1u)) << lo) : 0u;
        }
        if (MK == 1 || __any_sync(0xffffffffu, col_lo > 0 || col_hi < 32)) {
#pragma unroll
          for (int x = 0; x < 16; ++x) pair(x, IntC<1>{});
        } else {
#pragma unroll
          for (int x = 0; x < 16; ++x) pair(x, IntC<0>{});
        }
        // The products of the sub-tile that used this result buffer last must have read it.
        const int ob = g % C::N_OBUF, use = g / C::N_OBUF;
        if (use > 0 && !mbar_wait(out_free + ob, (use - 1) & 1, ab, kAbortBwdPFull)) {
          alive = false;
          break;
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {  // chunk 4 wg + c = this group's queries 8c .. 8c+7
          const uint32_t off = out_row + ob * C::OBUF_BYTES + (((uint32_t)(4 * wg + c) ^ sw) << 4);
          sts_v4(off + C::OUT_GS * C::OUT_BYTES, pk_gs[4 * c], pk_gs[4 * c + 1], pk_gs[4 * c + 2], pk_gs[4 * c + 3]);
          if constexpr (HAS_GT) sts_v4(off + C::OUT_GT * C::OUT_BYTES, pk_gt[4 * c], pk_gt[4 * c + 1], pk_gt[4 * c + 2], pk_gt[4 * c + 3]);
        }
        // A and P go to their TMEM columns (this group's 32 queries = 16 packed columns) once the previous
        // sub-tile's dV products have read them
        if (g > 0 && !mbar_wait(av_free, (g - 1) & 1, ab, kAbortBwdPFull)) {
          alive = false;
          break;
        }
        {
          const uint32_t trow = tmem + ((uint32_t)(quarter * 32) << 16) + 16 * wg;
          if constexpr (HAS_GT) tmem_st16(trow + C::COL_AV, pk_av);
          if constexpr (HAS_GO) tmem_st16(trow + C::COL_P, pk_p);
          tmem_wait_st();
        }
        fence_async_smem();
        tc_fence_before();
        mbar_arrive(p_full + (g & 1));
      }
      if (!alive) break;
      // item epilogue: group 0 stores dK, group 1 dV
      if (!mbar_wait(done, kact & 1, ab, kAbortBwdDone)) break;
      tc_fence_after();
      {
        uint32_t r0[32], r1[32];
        const uint32_t src = tmem + ((uint32_t)(quarter * 32) << 16) + (wg == 0 ? C::COL_DK : C::COL_DV);
        tmem_ld32(src, r0);
        tmem_ld32(src + 32, r1);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(acc_free);
        store_row(wg == 0 ? a.dk : a.dv, it.bh, own_idx, r0, r1, wg == 0 ? a.sm_scale : 1.f);
      }
      ++kact;
    }
  } else {
    // ------------------------------------------------------------------ dQ read-back
    const int quarter = warp & 3;
    const uint32_t tbase = tmem + ((uint32_t)(quarter * 32) << 16) + C::COL_DQ;
    const uint32_t dqs = smem_u32(smem + C::OFF_DQS);
    int g = 0;
    bool alive = true;
    FItem it;
    // The 128 threads meet at a hardware barrier.  That is safe although it has no time limit: every decision to leave
    // the loop is taken from rb_ok, which one thread writes before a meeting and all read after it, so nobody can be
    // missing at the next one; and nothing between two meetings waits on another role.
    auto rb_meet = [&]() { asm volatile("bar.sync 1, 128;" ::: "memory"); };
    for (int k = 0; alive && k < k_max; ++k) {
      if (!get_item(k, it) || it.n_sub == 0) continue;
      for (int s = 0; s < it.n_sub; ++s, ++g) {
        // one thread polls for the warpgroup (every polling warp is traffic on the shared-memory port)
        if (tid == 384) *rb_ok = mbar_wait(dq_full, g & 1, ab, kAbortBwdDone) ? 1 : 0;
        rb_meet();
        if (*rb_ok == 0) {
          alive = false;
          break;
        }
        tc_fence_after();
        uint32_t r0[32], r1[32];
        tmem_ld32(tbase, r0);
        tmem_ld32(tbase + 32, r1);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(dq_free);
        // An M = 64 accumulator: row 16 * quarter + l of the sub-tile is in lane l < 16 of this quarter.  The tile goes
        // to a staging area in shared memory and from there to the accumulation buffer as two TMA reductions (one
        // instruction each, coalesced and asynchronous) instead of sixteen vector reductions per thread.
        if (g > 0) {  // the previous sub-tile's reductions must have read the staging area
          if (tid == 384) bulk_wait_read();
          rb_meet();
        }
        if (lane < 16) {
          const int r = 16 * quarter + lane;
          const uint32_t rowa = dqs + r * 128, sw = (uint32_t)(r & 7);
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            sts_v4(rowa + (((uint32_t)c ^ sw) << 4), r0[4 * c], r0[4 * c + 1], r0[4 * c + 2], r0[4 * c + 3]);
            sts_v4(rowa + 8192 + (((uint32_t)c ^ sw) << 4), r1[4 * c], r1[4 * c + 1], r1[4 * c + 2], r1[4 * c + 3]);
          }
        }
        fence_async_smem();
        rb_meet();
        if (tid == 384) {
          const int i0 = it.loop_begin + s * BL;
          tma_reduce_add_4d(&maps.dq, dqs, 0, i0, it.h, it.b);
          tma_reduce_add_4d(&maps.dq, dqs + 8192, 32, i0, it.h, it.b);
          bulk_commit();
        }
      }
    }
    if (tid == 384) bulk_wait_all();  // the reductions must have landed (and read shared memory) before the CTA ends
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

// dq = T(dq_acc * scale), 8 elements per thread
template <typename T>
__global__ void dq_convert_kernel(const float* __restrict__ acc, T* __restrict__ dq, long long n8, float scale) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  const float4 lo = reinterpret_cast<const float4*>(acc)[2 * i], hi = reinterpret_cast<const float4*>(acc)[2 * i + 1];
  reinterpret_cast<uint4*>(dq)[i] = make_uint4(Elem<T>::pack(lo.x * scale, lo.y * scale), Elem<T>::pack(lo.z * scale, lo.w * scale),
                                               Elem<T>::pack(hi.x * scale, hi.y * scale), Elem<T>::pack(hi.z * scale, hi.w * scale));
}

static int fused_sm_count() {
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

template <typename T, bool HAS_GO, bool HAS_GT, int MK>
static int launch_fused64(const jvpfa_bwd_args& a, cudaStream_t stream) {
  using C = BwdFCfg<HAS_GO, HAS_GT>;
  int* status = tc5_status_device_ptr();
  if (!status) {
    set_last_cuda_error(cudaErrorUnknown, "status word address");
    return JVPFA_ERR_CUDA;
  }
  BwdFMaps m;
  const CUtensorMapDataType dt = Fmt<T>::kTma;
  const int64_t* st = a.in_stride;
  bool ok = encode_map4(&m.k, dt, a.k, a.L, a.H, a.B, st, C::OWN) && encode_map4(&m.v, dt, a.v, a.L, a.H, a.B, st, C::OWN) &&
            encode_map4(&m.q, dt, a.q, a.L, a.H, a.B, st, C::BL);
  m.tk = m.tv = m.k;
  m.go = m.tq = m.g = m.q;
  if (HAS_GO) ok = ok && encode_map4(&m.go, dt, a.go, a.L, a.H, a.B, nullptr, C::BL);
  if (HAS_GT)
    ok = ok && encode_map4(&m.tk, dt, a.tk, a.L, a.H, a.B, st, C::OWN) && encode_map4(&m.tv, dt, a.tv, a.L, a.H, a.B, st, C::OWN) &&
         encode_map4(&m.tq, dt, a.tq, a.L, a.H, a.B, st, C::BL) && encode_map4(&m.g, dt, a.gto, a.L, a.H, a.B, nullptr, C::BL);
  ok = ok && encode_map4d_f32(&m.dq, a.dq_accum, C::D, a.L, a.H, a.B, C::BL);
  if (!ok) {
    set_last_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled(bwd fused64)");
    return JVPFA_ERR_CUDA;
  }
  const int sms = fused_sm_count();
  if (sms <= 0) {
    set_last_cuda_error(cudaErrorUnknown, "multiprocessor count");
    return JVPFA_ERR_CUDA;
  }
  const size_t n = (size_t)a.B * a.H * a.L * 64;
  cudaError_t e = cudaMemsetAsync(a.dq_accum, 0, n * sizeof(float), stream);
  if (e != cudaSuccess) {
    set_last_cuda_error(e, "cudaMemsetAsync(dq_accum)");
    return JVPFA_ERR_CUDA;
  }
  auto kern = bwd_tc5_fused64_kernel<T, HAS_GO, HAS_GT, MK>;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
  if (e != cudaSuccess) {
    set_last_cuda_error(e, "cudaFuncSetAttribute(bwd_tc5_fused64)");
    return JVPFA_ERR_CUDA;
  }
  const long long n_items = (long long)((a.L + C::OWN - 1) / C::OWN) * a.B * a.H;
  const int grid = (int)(n_items < sms ? n_items : sms);
  kern<<<grid, C::NTHREADS, C::SMEM_BYTES, stream>>>(a, m, a.dq_accum, status);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_cuda_error(e, "launch bwd_tc5_fused64");
    return JVPFA_ERR_CUDA;
  }
  const long long n8 = (long long)(n / 8);
  dq_convert_kernel<T><<<(unsigned)((n8 + 255) / 256), 256, 0, stream>>>(a.dq_accum, reinterpret_cast<T*>(a.dq), n8, a.sm_scale);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_cuda_error(e, "launch dq_convert");
    return JVPFA_ERR_CUDA;
  }
  return JVPFA_OK;
}

template <typename T>
static int launch_fused64_t(const jvpfa_bwd_args& a, cudaStream_t s) {
  const bool go = a.go != nullptr, gt = a.gto != nullptr;
  if (a.mask.kind == JVPFA_MASK_BIAS) return launch_fused64<T, true, false, 2>(a, s);  // eligible only through O alone
  if (a.mask.kind == JVPFA_MASK_BOOL) {
    if (go && gt) return launch_fused64<T, true, true, 1>(a, s);
    if (gt) return launch_fused64<T, false, true, 1>(a, s);
    return launch_fused64<T, true, false, 1>(a, s);
  }
  if (go && gt) return launch_fused64<T, true, true, 0>(a, s);
  if (gt) return launch_fused64<T, false, true, 0>(a, s);
  return launch_fused64<T, true, false, 0>(a, s);
}

}  // namespace tc5

// The single-pass kernel serves D = 64 with index masks (none, causal, key padding) and boolean masks that come without
// tile bitmaps, when the caller provides the fp32 accumulation buffer for dQ.
bool bwd_tc5_fused64_eligible(const jvpfa_bwd_args& a) {
  if (a.D != 64 || a.dq_accum == nullptr) return false;
  if ((reinterpret_cast<uintptr_t>(a.dq_accum) & 15u) != 0) return false;
  const int k = a.mask.kind;
  // A boolean mask without tile bitmaps (dense, or not looked at beforehand): with them the two-launch kernels, which
  // step over dead tiles, are the better choice.
  if (k == JVPFA_MASK_BOOL) return a.mask_tile_live == nullptr && a.mask_tile_live_t == nullptr;
  // An additive bias of the tensors' type: only the backward through O alone has the registers for it.
  if (k == JVPFA_MASK_BIAS) return a.gto == nullptr && a.mask.bias_dtype == a.dtype;
  return k == JVPFA_MASK_NONE || k == JVPFA_MASK_CAUSAL || k == JVPFA_MASK_KVLEN;
}

int launch_bwd_tc5_fused64(const jvpfa_bwd_args& a, cudaStream_t s) {
  return a.dtype == JVPFA_BF16 ? tc5::launch_fused64_t<__nv_bfloat16>(a, s) : tc5::launch_fused64_t<__half>(a, s);
}

}  // namespace jvpfa
