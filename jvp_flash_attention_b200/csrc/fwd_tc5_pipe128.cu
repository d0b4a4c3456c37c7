// Fused primal (+ tangent) attention forward for head dimension 128, bf16 / fp16, on the Blackwell tensor cores,
// with the score products of the next key tile running under the softmax of the current one.
//
// CTA = one 128-row query tile of one (batch, head); 6 warps:
//   warp 0      TMA producer (one lane) and owner of the TMEM allocation
//   warp 1      MMA issuer (one lane)
//   warps 2..5  softmax / correction / epilogue: thread <-> one query row <-> one TMEM lane
// TMEM columns (fp32): two score buffers [S | tS] of 128 columns (64 without tangents), then O [128] | tO' [128];
//   P (16 bit, 32 columns) overwrites the head of S and W = P*tS*scale the head of tS; both feed the output MMAs
//   straight from TMEM as the A operand.
// Shared memory: Q, tQ resident; a ring of two [K | tK] stages and a ring of two [V | tV] stages, released
//   separately: the keys of a stage are free again as soon as its scores exist, long before its values are.
// The issuer's order is  S(0), S(1), PV(0), S(2), PV(1), ...: the tensor pipe executes in issue order, so S(t+2)
// overwrites score buffer t & 1 only after PV(t) has read P(t) and W(t) from it, and no barrier is needed for that.
// Per key tile (the products that share an operand are single instructions over adjacent tiles):
//   [S | Q tK^T] = Q [K | tK]^T  (N = 128) ;  tS += tQ K^T  (N = 64)                      -> commit(s_full[buf])
//   softmax: lazy running max (O, tO' rescaled only when the max grows by more than 2^8, after the previous
//            tile's output MMAs have landed); P = 2^(x-m); l += sum P; mu += sum W           -> arrive(p_full[buf])
//   [O | tO'] += P [V | tV]  (N = 256) ;  tO' += W V  (N = 128)                     -> commit(v_empty, pv_done)
// Epilogue: O = O/l ; tO = tO'/l - (mu/l) O ; lse = m + log2 l  (same quantities as the register-tiled kernel in
// fwd_generic.cu, which follows jvp_attention.py:125-336, 1011-1033).
// Every wait is bounded; a wait that gives up sets the CTA's abort flag and the device status word, the CTA's rows
// get lse = NaN, and the teardown still runs.
#include "tc5_common.cuh"

namespace jvpfa {
namespace tc5 {

template <bool DUAL>
struct FwdPipeCfg {
  static constexpr int D = 128;
  static constexpr int BM = 128;
  static constexpr int BN = 64;
  static constexpr int STAGES = 2;
  static constexpr int NTHREADS = 192;
  static constexpr int Q_BYTES = BM * D * 2;        // 32 KiB: two 64-column halves of 16 KiB
  static constexpr int HALF_BYTES = BN * 64 * 2;    // 8 KiB: 64 keys x 64 columns
  static constexpr int N_T = DUAL ? 2 : 1;          // primal, tangent
  static constexpr int K_STAGE = N_T * 2 * HALF_BYTES;  // [K h0][tK h0][K h1][tK h1]
  static constexpr int V_STAGE = N_T * 2 * HALF_BYTES;  // [V h0][V h1][tV h0][tV h1]
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = N_T * Q_BYTES;
  static constexpr int OFF_V = OFF_K + STAGES * K_STAGE;
  // the live key tiles of the CTA's query tile, in order (boolean masks with a tile bitmap: the others are not visited)
  static constexpr int MAX_KEY_TILES = 1024;
  static constexpr int OFF_IDS = OFF_V + STAGES * V_STAGE;
  static constexpr int TILE_BYTES = OFF_IDS + MAX_KEY_TILES * 2;
  static constexpr int SMEM_BYTES = TILE_BYTES + 256 /*barriers*/ + 1024 /*alignment slack*/;
  static constexpr int SC_COLS = DUAL ? 2 * BN : BN;  // one score buffer
  static constexpr int COL_O = 2 * SC_COLS;
  static constexpr int COL_TO = COL_O + D;
  static constexpr int COLS_ALLOC = DUAL ? 512 : 256;
};

struct FwdPipeMaps {
  CUtensorMap q, tq, k, tk, v, tv;
};

// MK: 0 = none / causal / key padding; 1 = uint8 mask; 2 = bias of the element type T (the softmax thread of a
// query row reads its 64 mask elements of the tile with 16-byte loads before it waits for the scores; key stride 1,
// 16-byte aligned rows and L % 16 == 0 are the host's responsibility); 3 = uint8 mask with the bitmap of 128 x 64
// tiles that hold a true entry (jvpfa_mask_tiles): the CTA lists its query tile's live key tiles once and every role
// walks that list, so tiles without a true entry are neither loaded nor multiplied.
template <typename T, bool DUAL, int MK>
__global__ void __launch_bounds__(192, 1)
fwd_tc5_pipe128_kernel(const jvpfa_fwd_args a, const __grid_constant__ FwdPipeMaps maps, int* status) {
  using C = FwdPipeCfg<DUAL>;
  constexpr int D = C::D, BM = C::BM, BN = C::BN, STAGES = C::STAGES;
  const bool dead_on_entry = *(volatile int*)status != 0;  // an earlier bounded wait gave up

  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  unsigned char* smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  unsigned char* sQ = smem + C::OFF_Q;
  unsigned char* sTQ = sQ + C::Q_BYTES;  // DUAL only
  unsigned char* sK = smem + C::OFF_K;
  unsigned char* sV = smem + C::OFF_V;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::TILE_BYTES);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* k_empty = bars + 3;   // [2]
  uint64_t* v_full = bars + 5;    // [2]
  uint64_t* v_empty = bars + 7;   // [2]
  uint64_t* s_full = bars + 9;    // [2]
  uint64_t* p_full = bars + 11;   // [2]
  uint64_t* pv_done = bars + 13;  // one phase per key tile
  uint64_t* o_full = bars + 14;   // all output MMAs of the CTA have landed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* n_live = reinterpret_cast<int*>(tmem_slot + 2);  // MK == 3: length of the list
  const unsigned short* ids = reinterpret_cast<const unsigned short*>(smem + C::OFF_IDS);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int L = a.L;
  const int bh = blockIdx.y;
  const int tma_b = bh / a.H, tma_h = bh - tma_b * a.H;  // coordinates in the (D, L, H, B) tensor maps
  const int mt = (int)gridDim.x - 1 - (int)blockIdx.x;   // heaviest causal tiles first
  const int m0 = mt * BM;
  const bool causal = a.mask.kind == JVPFA_MASK_CAUSAL;
  int n_valid = L;  // keys j < n_valid can attend (before the causal rule)
  if (a.mask.kind == JVPFA_MASK_KVLEN) {
    const int n = a.mask.kv_len[tma_b];
    n_valid = n < 0 ? 0 : (n > L ? L : n);
  }
  int n_end = n_valid;
  if (causal) n_end = min(n_end, m0 + BM);
  int n_tiles = (n_end + BN - 1) / BN;
  // key tile visited at step t
  auto key_tile = [&](int t) -> int {
    if constexpr (MK == 3) return (int)ids[t];
    return t;
  };

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
      mbar_init(k_full + s, 1);
      mbar_init(k_empty + s, 1);
      mbar_init(v_full + s, 1);
      mbar_init(v_empty + s, 1);
      mbar_init(s_full + s, 1);
      mbar_init(p_full + s, 128);
    }
    mbar_init(pv_done, 1);
    mbar_init(o_full, 1);
    *abort_flag = 0;
    fence_mbar_init();
    if constexpr (MK == 3) {
      // the bitmap has the mask's own extents: broadcast dimensions (stride 0) have one entry
      const int n_q_tiles = (L + BM - 1) / BM, n_words = ((L + BN - 1) / BN + 63) >> 6;
      const long long hm = (a.mask.stride[0] ? (long long)tma_b * (a.mask.stride[1] ? a.H : 1) : 0) +
                           (a.mask.stride[1] ? tma_h : 0);
      const long long qm = a.mask.stride[2] ? hm * n_q_tiles + mt : hm;
      const unsigned long long* live = reinterpret_cast<const unsigned long long*>(a.mask_tile_live) + qm * n_words;
      unsigned short* out = reinterpret_cast<unsigned short*>(smem + C::OFF_IDS);
      int cnt = 0;
      for (int w = 0; w * 64 < n_tiles; ++w) {
        unsigned long long bits = __ldg(live + w);
        const int rem = n_tiles - 64 * w;
        if (rem < 64) bits &= (1ull << rem) - 1ull;
        while (bits) {
          out[cnt++] = (unsigned short)(64 * w + __ffsll((long long)bits) - 1);
          bits &= bits - 1ull;
        }
      }
      *n_live = cnt;
    }
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

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && n_tiles > 0) {
      prefetch_tmap(&maps.q);
      prefetch_tmap(&maps.k);
      prefetch_tmap(&maps.v);
      mbar_expect_tx(q_full, C::N_T * C::Q_BYTES);
      for (int hf = 0; hf < 2; ++hf) {
        tma_load_4d(sQ + hf * (BM * 128), &maps.q, q_full, hf * 64, m0, tma_h, tma_b);
        if constexpr (DUAL) tma_load_4d(sTQ + hf * (BM * 128), &maps.tq, q_full, hf * 64, m0, tma_h, tma_b);
      }
      auto load_k = [&](int t) -> bool {
        const int st = t & 1;
        if (!mbar_wait(k_empty + st, ((t >> 1) & 1) ^ 1, ab, kAbortKvEmpty)) return false;
        unsigned char* base = sK + st * C::K_STAGE;
        mbar_expect_tx(k_full + st, C::K_STAGE);
        for (int hf = 0; hf < 2; ++hf) {
          tma_load_4d(base + hf * C::N_T * C::HALF_BYTES, &maps.k, k_full + st, hf * 64, key_tile(t) * BN, tma_h, tma_b);
          if constexpr (DUAL)
            tma_load_4d(base + (hf * 2 + 1) * C::HALF_BYTES, &maps.tk, k_full + st, hf * 64, key_tile(t) * BN, tma_h, tma_b);
        }
        return true;
      };
      auto load_v = [&](int t) -> bool {
        const int st = t & 1;
        if (!mbar_wait(v_empty + st, ((t >> 1) & 1) ^ 1, ab, kAbortKvEmpty)) return false;
        unsigned char* base = sV + st * C::V_STAGE;
        mbar_expect_tx(v_full + st, C::V_STAGE);
        for (int hf = 0; hf < 2; ++hf) {
          tma_load_4d(base + hf * C::HALF_BYTES, &maps.v, v_full + st, hf * 64, key_tile(t) * BN, tma_h, tma_b);
          if constexpr (DUAL)
            tma_load_4d(base + (2 + hf) * C::HALF_BYTES, &maps.tv, v_full + st, hf * 64, key_tile(t) * BN, tma_h, tma_b);
        }
        return true;
      };
      // Stages come free in the order S(t) done, PV(t-1) done, S(t+1) done, ...: the loads are requested in it.
      bool ok = load_k(0);
      if (ok && n_tiles > 1) ok = load_k(1);
      for (int t = 0; ok && t < n_tiles; ++t) {
        ok = load_v(t);
        if (ok && t + 2 < n_tiles) ok = load_k(t + 2);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idesc_s1 = make_idesc(Fmt<T>::kIdesc, BM, BN, 0, 0);      // 128 x 64
      constexpr uint32_t idesc_s2 = make_idesc(Fmt<T>::kIdesc, BM, 2 * BN, 0, 0);  // 128 x 128: [S | Q tK^T]
      constexpr uint32_t idesc_o1 = make_idesc(Fmt<T>::kIdesc, BM, D, 0, 1);       // 128 x 128, B MN-major
      constexpr uint32_t idesc_o2 = make_idesc(Fmt<T>::kIdesc, BM, 2 * D, 0, 1);   // 128 x 256: [O | tO']
      // Shared-memory descriptors as low words (tc5_common.cuh): the high word is the same for every tile used here and
      // stepping through a tile is an integer add, which keeps the issuing thread's own instruction count small.
      // K-major operands: contraction step ks over D = 32 bytes inside a 64-column half.  MN-major [V | tV]: contraction
      // step kk over the keys = 2048 bytes; the 64-column chunks are HALF_BYTES apart (the leading offset).
      const uint32_t q_lo = kDescLo | (smem_u32(sQ) >> 4), tq_lo = kDescLo | (smem_u32(sTQ) >> 4);
      constexpr uint32_t kVLo = (uint32_t)(C::HALF_BYTES >> 4) << 16;
      auto k_off = [](uint32_t half, int ks) -> uint32_t { return (uint32_t)((ks >> 2) * half + (ks & 3) * 32) >> 4; };
      constexpr uint32_t QH = BM * 128, KH = C::N_T * C::HALF_BYTES;
      auto issue_s = [&](int t) -> bool {
        const int st = t & 1;
        if (!mbar_wait(k_full + st, (t >> 1) & 1, ab, kAbortKvFull)) return false;
        tc_fence_after();
        const uint32_t k_lo = kDescLo | (smem_u32(sK + st * C::K_STAGE) >> 4);
        const uint32_t sc = tmem + st * C::SC_COLS;
        umma_ss_lo<false>(sc, q_lo, k_lo, DUAL ? idesc_s2 : idesc_s1);
#pragma unroll
        for (int ks = 1; ks < 8; ++ks)
          umma_ss_lo<true>(sc, q_lo + k_off(QH, ks), k_lo + k_off(KH, ks), DUAL ? idesc_s2 : idesc_s1);
        if constexpr (DUAL) {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            umma_ss_lo<true>(sc + BN, tq_lo + k_off(QH, ks), k_lo + k_off(KH, ks), idesc_s1);
        }
        tc_commit(s_full + st);
        tc_commit(k_empty + st);
        return true;
      };
      bool ok = mbar_wait(q_full, 0, ab, kAbortQFull);
      if (ok) ok = issue_s(0);
      for (int t = 0; ok && t < n_tiles; ++t) {
        if (t + 1 < n_tiles && !issue_s(t + 1)) break;
        const int st = t & 1;
        const uint32_t ph = (t >> 1) & 1;
        if (!mbar_wait(p_full + st, ph, ab, kAbortPFull)) break;
        if (!mbar_wait(v_full + st, ph, ab, kAbortKvFull)) break;
        tc_fence_after();
        const uint32_t v_lo = kVLo | (smem_u32(sV + st * C::V_STAGE) >> 4);
        const uint32_t sc = tmem + st * C::SC_COLS;
        umma_ts_lo_dyn(tmem + C::COL_O, sc, v_lo, DUAL ? idesc_o2 : idesc_o1, t > 0);
#pragma unroll
        for (int kk = 1; kk < 4; ++kk)
          umma_ts_lo<true>(tmem + C::COL_O, sc + kk * 8, v_lo + kk * 128, DUAL ? idesc_o2 : idesc_o1);
        if constexpr (DUAL) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) umma_ts_lo<true>(tmem + C::COL_TO, sc + BN + kk * 8, v_lo + kk * 128, idesc_o1);
        }
        tc_commit(v_empty + st);
        tc_commit(pv_done);
      }
      tc_commit(o_full);
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue
    const int quarter = warp & 3;         // TMEM lane quarter this warp may access
    const int row = quarter * 32 + lane;  // tile row == TMEM lane
    const int i = m0 + row;               // query index
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t tO = tmem + lane_off + C::COL_O, tTO = tmem + lane_off + C::COL_TO;
    const float scale_log2 = a.sm_scale * kLog2e;
    const float2 c2 = make_float2(scale_log2, scale_log2);
    const float2 sc2 = make_float2(a.sm_scale, a.sm_scale);
    float m_used = -INFINITY, l_run = 0.f, mu_run = 0.f;
    bool alive = true;

    constexpr bool BOOLM = MK == 1 || MK == 3;
    constexpr int MESZ = BOOLM ? 1 : 2;        // bytes per mask element
    constexpr int MW = MK == 0 ? 1 : 16 * MESZ;  // 32-bit words per row of a 64-key tile
    const unsigned char* mrow = nullptr;
    if constexpr (MK != 0)
      mrow = reinterpret_cast<const unsigned char*>(a.mask.ptr) +
             ((long long)tma_b * a.mask.stride[0] + (long long)tma_h * a.mask.stride[1] +
              (long long)min(i, L - 1) * a.mask.stride[2]) * MESZ;

    for (int t = 0; t < n_tiles; ++t) {
      const int n0 = key_tile(t) * BN;
      const int st = t & 1;
      const uint32_t tS = tmem + lane_off + st * C::SC_COLS, tTS = tS + BN;
      uint32_t mw[MW];
      if constexpr (MK != 0) {  // issued before the wait: the loads fly while the scores are formed
#pragma unroll
        for (int q4 = 0; q4 < MW / 4; ++q4) {
          uint4 r = make_uint4(0u, 0u, 0u, 0u);
          if (n0 + (q4 + 1) * (16 / MESZ) <= L) r = ldg_nc_v4(mrow + (size_t)n0 * MESZ + 16 * q4);
          mw[4 * q4] = r.x, mw[4 * q4 + 1] = r.y, mw[4 * q4 + 2] = r.z, mw[4 * q4 + 3] = r.w;
        }
      }
      if (!mbar_wait(s_full + st, (t >> 1) & 1, ab, kAbortSFull)) {
        alive = false;
        break;
      }
      tc_fence_after();
      uint32_t x0[32], x1[32];
      tmem_ld32(tS, x0);
      tmem_ld32(tS + 32, x1);
      tmem_wait_ld();
      // live key columns of this row inside the tile: col < col_hi
      int col_hi = min(BN, n_valid - n0);
      if (causal) col_hi = min(col_hi, i - n0 + 1);
      const bool partial = (n0 + BN > n_valid) || (causal && n0 + BN - 1 > m0);
      // Row maximum of the tile in log2 units.  Without a mask or bias and with a positive scale it is taken over
      // the raw scores and the scaling is folded into the exponent's multiply-add; otherwise the scores are scaled,
      // biased and masked first.
      const bool raw_max = MK == 0 && a.sm_scale > 0.f;
      float mx;
      if (raw_max) {
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
      if (t > 0 && __any_sync(0xffffffffu, grow)) {
        // O / tO' are rescaled in place: the previous tile's output MMAs must have landed.  This tile's cannot have
        // been issued yet (they wait for this thread's arrival below), so the barrier is at most one phase ahead.
        if (!mbar_wait(pv_done, (t - 1) & 1, ab, kAbortOFull)) {
          alive = false;
          break;
        }
        tc_fence_after();
        const float2 al2 = make_float2(alpha, alpha);
#pragma unroll
        for (int c = 0; c < (DUAL ? 2 : 1) * D / 32; ++c) {  // tO' follows O
          uint32_t r[32];
          tmem_ld32(tO + 32 * c, r);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const float2 v = __fmul2_rn(pf2(r[2 * e], r[2 * e + 1]), al2);
            r[2 * e] = __float_as_uint(v.x), r[2 * e + 1] = __float_as_uint(v.y);
          }
          tmem_st32(tO + 32 * c, r);
        }
      }
      // Exponentials, row sums, W = P * tS * scale and the packing to 16 bit in one loop per half tile, so that the
      // special-function unit's latency is covered by the arithmetic of the neighbouring columns.
      const float2 nm2 = make_float2(-m_eff, -m_eff);
      float2 ls2 = make_float2(0.f, 0.f), ms2 = make_float2(0.f, 0.f);
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        uint32_t* xs = hh ? x1 : x0;
        uint32_t tt[DUAL ? 32 : 1];
        uint32_t pp[16], wp[DUAL ? 16 : 1];
        if constexpr (DUAL) {
          tmem_ld32(tTS + 32 * hh, tt);
          tmem_wait_ld();
        }
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          float2 e;
          if (raw_max)
            e = __ffma2_rn(pf2(xs[2 * c], xs[2 * c + 1]), c2, nm2);
          else
            e = __fadd2_rn(pf2(xs[2 * c], xs[2 * c + 1]), nm2);
          const float2 pv = make_float2(fast_exp2(e.x), fast_exp2(e.y));
          ls2 = __fadd2_rn(ls2, pv);
          pp[c] = Elem<T>::pack(pv.x, pv.y);
          if constexpr (DUAL) {
            const float2 w = __fmul2_rn(pv, __fmul2_rn(pf2(tt[2 * c], tt[2 * c + 1]), sc2));
            ms2 = __fadd2_rn(ms2, w);
            wp[c] = Elem<T>::pack(w.x, w.y);
          }
        }
        // Packed columns 16 hh .. 16 hh + 15 of P (over S, already in registers) and of W (over tS: with hh = 0 they
        // cover fp32 columns 0..15 of tS, read above; the second half, columns 32..63, is read before columns 16..31
        // are written).
        tmem_st16(tS + 16 * hh, pp);
        if constexpr (DUAL) tmem_st16(tTS + 16 * hh, wp);
      }
      l_run = l_run * alpha + (ls2.x + ls2.y);
      if constexpr (DUAL) mu_run = mu_run * alpha + (ms2.x + ms2.y);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(p_full + st);
    }

    // ---- epilogue ----
    // (pv_done cannot serve here: a thread that leaves the loop may be two of its phases behind.)
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

template <typename T, bool DUAL, int MK>
static int launch_pipe128(const jvpfa_fwd_args& a, cudaStream_t stream) {
  using C = FwdPipeCfg<DUAL>;
  int* status = tc5_status_device_ptr();
  if (!status) {
    set_last_cuda_error(cudaErrorUnknown, "status word address");
    return JVPFA_ERR_CUDA;
  }
  FwdPipeMaps maps;
  const CUtensorMapDataType dt = Fmt<T>::kTma;
  auto enc = [&](CUtensorMap* m, const void* p, int rows) {
    return encode_map4d(m, dt, p, C::D, a.L, a.H, a.B, a.in_stride, rows);
  };
  bool ok = enc(&maps.q, a.q, C::BM) && enc(&maps.k, a.k, C::BN) && enc(&maps.v, a.v, C::BN);
  if (DUAL)
    ok = ok && enc(&maps.tq, a.tq, C::BM) && enc(&maps.tk, a.tk, C::BN) && enc(&maps.tv, a.tv, C::BN);
  else
    maps.tq = maps.tk = maps.tv = maps.q;
  if (!ok) {
    set_last_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled");
    return JVPFA_ERR_CUDA;
  }
  auto kern = fwd_tc5_pipe128_kernel<T, DUAL, MK>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
  if (e != cudaSuccess) {
    set_last_cuda_error(e, "cudaFuncSetAttribute(fwd_tc5_pipe128)");
    return JVPFA_ERR_CUDA;
  }
  dim3 grid((a.L + C::BM - 1) / C::BM, a.B * a.H);
  kern<<<grid, C::NTHREADS, C::SMEM_BYTES, stream>>>(a, maps, status);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_cuda_error(e, "launch fwd_tc5_pipe128");
    return JVPFA_ERR_CUDA;
  }
  return JVPFA_OK;
}

template <typename T>
static int launch_pipe128_t(const jvpfa_fwd_args& a, cudaStream_t s) {
  const bool dual = a.tq != nullptr;
  if (a.mask.kind == JVPFA_MASK_BOOL && a.mask_tile_live != nullptr && (a.L + 63) / 64 <= FwdPipeCfg<true>::MAX_KEY_TILES)
    return dual ? launch_pipe128<T, true, 3>(a, s) : launch_pipe128<T, false, 3>(a, s);
  if (a.mask.kind == JVPFA_MASK_BOOL) return dual ? launch_pipe128<T, true, 1>(a, s) : launch_pipe128<T, false, 1>(a, s);
  if (a.mask.kind == JVPFA_MASK_BIAS) return dual ? launch_pipe128<T, true, 2>(a, s) : launch_pipe128<T, false, 2>(a, s);
  return dual ? launch_pipe128<T, true, 0>(a, s) : launch_pipe128<T, false, 0>(a, s);
}

}  // namespace tc5

int launch_fwd_tc5_pipe128(const jvpfa_fwd_args& a, cudaStream_t s) {
  return a.dtype == JVPFA_BF16 ? tc5::launch_pipe128_t<__nv_bfloat16>(a, s) : tc5::launch_pipe128_t<__half>(a, s);
}

}  // namespace jvpfa
