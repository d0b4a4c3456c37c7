// Backward of <gO, O> + <gtO, tO> for bf16 / fp16 on tcgen05 tensor cores (TMA + TMEM).
//
// Same split as the register-tiled backward (bwd_generic.cu; upstream jvp_attention.py:2008-2233):
// one launch owns 128-key tiles and loops over query tiles (dK, dV), one owns 128-query tiles and
// loops over key tiles (dQ).  Both are instances of one kernel template:
//
//   "own" side  : 128 rows, one per TMEM lane and per softmax thread, operand tiles resident in smem
//   "loop" side : 64-column tiles streamed through a TMA ring
//
// Per tile the MMA warp forms up to four 128x64 fp32 score accumulators in TMEM
//     S  = own.(K|Q) loop.(Q|K)^T          TS = tangent scores (two MMAs)
//     E  = own.(V|G) loop.(G|V)^T          FP = F (+ dP)   (one or two MMAs)
// the softmax threads turn them, 16 columns at a time, into the 16-bit operands
//     P, A = P*(tS-mu), gtS = P*(E-eps), gS = P*((E-eps)*(tS-mu) + FP - delta - rowsum(G*tO))
// written back over the accumulators they came from, and a second group of MMAs (A operand
// from TMEM, B = the streamed tile used MN-major) accumulates dK/dV or dQ in TMEM.
// Formulas: see bwd_generic.cu.  All waits are bounded (tc5_common.cuh).
#include "tc5_common.cuh"

namespace jvpfa {
namespace tc5 {

struct BwdMaps {
  CUtensorMap k, v, tk, tv;   // key-side tensors
  CUtensorMap q, go, tq, g;   // query-side tensors (g = cotangent of tO)
};

template <int D, bool OWN_KEYS, bool HAS_GO, bool HAS_GT>
struct BwdCfg {
  static constexpr int OWN = 128;
  static constexpr int BL = 64;
  static constexpr int NTHREADS = 192;
  static constexpr int N_KEY_TILES = HAS_GT ? 4 : 2;                       // K, V, tK, tV
  static constexpr int N_QRY_TILES = 1 + (HAS_GO ? 1 : 0) + (HAS_GT ? 2 : 0);  // Q, gO, tQ, G
  static constexpr int N_OWN = OWN_KEYS ? N_KEY_TILES : N_QRY_TILES;
  static constexpr int N_LOOP = OWN_KEYS ? N_QRY_TILES : N_KEY_TILES;
  static constexpr int OWN_BYTES = OWN * D * 2;
  static constexpr int LOOP_BYTES = BL * D * 2;
  static constexpr int STAGES = (N_OWN * OWN_BYTES + 2 * N_LOOP * LOOP_BYTES <= 200 * 1024) ? 2 : 1;
  static constexpr int STAT_BYTES = OWN_KEYS ? STAGES * BL * 16 : 0;
  static constexpr int TILE_BYTES = N_OWN * OWN_BYTES + STAGES * N_LOOP * LOOP_BYTES;
  static constexpr int SMEM_BYTES = TILE_BYTES + STAT_BYTES + 256 + 1024;
  // TMEM columns
  static constexpr int NSC = HAS_GT ? 4 : 2;
  static constexpr int COL_S = 0;
  static constexpr int COL_TS = BL;                      // HAS_GT
  static constexpr int COL_E = 2 * BL;                   // HAS_GT
  static constexpr int COL_FP = HAS_GT ? 3 * BL : BL;
  static constexpr int COL_OUT0 = NSC * BL;              // dK (own keys) or dQ (own queries)
  static constexpr int COL_OUT1 = COL_OUT0 + D;          // dV (own keys only)
  static constexpr int COLS_USED = COL_OUT0 + (OWN_KEYS ? 2 * D : D);
  static constexpr int COLS_ALLOC = COLS_USED <= 128 ? 128 : (COLS_USED <= 256 ? 256 : 512);
  // tile slots inside the key-side / query-side groups
  static constexpr int SLOT_K = 0, SLOT_V = 1, SLOT_TK = 2, SLOT_TV = 3;
  static constexpr int SLOT_Q = 0, SLOT_GO = 1, SLOT_TQ = 1 + (HAS_GO ? 1 : 0), SLOT_G = 2 + (HAS_GO ? 1 : 0);
};

// MK: 0 = none / causal / key padding; 1 = uint8 mask; 2 = bias of the element type T.  For 1 and 2 the
// elementwise threads fetch the 16 mask elements of each column chunk from global memory ahead of the
// chunk's tcgen05.ld (own queries: one or two 16-byte loads of the thread's mask row; own keys: one element
// of each of 16 query rows).  Key stride 1, 16-byte aligned rows and L % 16 == 0 are the host's responsibility.
template <typename T, int D, bool OWN_KEYS, bool HAS_GO, bool HAS_GT, int MK>
__global__ void __launch_bounds__(192, 1)
bwd_tc5_kernel(const jvpfa_bwd_args a, const __grid_constant__ BwdMaps maps, int* status) {
  using C = BwdCfg<D, OWN_KEYS, HAS_GO, HAS_GT>;
  constexpr int OWN = C::OWN, BL = C::BL, STAGES = C::STAGES;
  constexpr int KSTEPS_D = D / 16;
  constexpr int KSTEPS_L = BL / 16;
  constexpr int HALVES = D / 64;

  // The own-queries launch that follows reads nothing this kernel writes: it is launched with programmatic
  // stream serialization and fills the SMs as this kernel's last CTAs leave them.
  if constexpr (OWN_KEYS) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const bool dead_on_entry = *(volatile int*)status != 0;  // an earlier bounded wait gave up

  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  unsigned char* smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  unsigned char* sOwn = smem;
  unsigned char* sLoop = smem + C::N_OWN * C::OWN_BYTES;
  float4* sStat = reinterpret_cast<float4*>(smem + C::TILE_BYTES);  // OWN_KEYS: [STAGES][BL] {lse, mu, eps, sub}
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::TILE_BYTES + C::STAT_BYTES);
  uint64_t* own_full = bars + 0;
  uint64_t* loop_full = bars + 1;            // [STAGES]
  uint64_t* loop_empty = bars + 1 + STAGES;  // [STAGES]
  uint64_t* s_full = bars + 1 + 2 * STAGES;
  uint64_t* p_full = s_full + 1;
  uint64_t* done = s_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_full + 3);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int L = a.L;
  const int bh = blockIdx.y;
  const int tma_b = bh / a.H, tma_h = bh - tma_b * a.H;  // coordinates in the (D, L, H, B) tensor maps
  const int b = bh / a.H;
  const bool causal = a.mask.kind == JVPFA_MASK_CAUSAL;
  int n_valid = L;
  if (a.mask.kind == JVPFA_MASK_KVLEN) {
    const int n = a.mask.kv_len[b];
    n_valid = n < 0 ? 0 : (n > L ? L : n);
  }
  // Tile ranges.  Own keys: heaviest (lowest) key tiles come first by construction; own queries:
  // reversed so that the heaviest (highest) query tiles start first.
  int own0, loop_begin, n_tiles;
  if constexpr (OWN_KEYS) {
    own0 = blockIdx.x * OWN;
    loop_begin = causal ? (own0 / BL) * BL : 0;
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
      mbar_init(loop_empty + s, 1);
    }
    mbar_init(s_full, 1);
    mbar_init(p_full, 128);
    mbar_init(done, 1);
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
    if (n_tiles > 0) {
      if (lane == 0) {
        mbar_expect_tx(own_full, C::N_OWN * C::OWN_BYTES);
        for (int hf = 0; hf < HALVES; ++hf) {
          const int x = hf * 64, o = hf * (OWN * 128);
          if constexpr (OWN_KEYS) {
            tma_load_4d(sOwn + C::SLOT_K * C::OWN_BYTES + o, &maps.k, own_full, x, own0, tma_h, tma_b);
            tma_load_4d(sOwn + C::SLOT_V * C::OWN_BYTES + o, &maps.v, own_full, x, own0, tma_h, tma_b);
            if constexpr (HAS_GT) {
              tma_load_4d(sOwn + C::SLOT_TK * C::OWN_BYTES + o, &maps.tk, own_full, x, own0, tma_h, tma_b);
              tma_load_4d(sOwn + C::SLOT_TV * C::OWN_BYTES + o, &maps.tv, own_full, x, own0, tma_h, tma_b);
            }
          } else {
            tma_load_4d(sOwn + C::SLOT_Q * C::OWN_BYTES + o, &maps.q, own_full, x, own0, tma_h, tma_b);
            if constexpr (HAS_GO) tma_load_4d(sOwn + C::SLOT_GO * C::OWN_BYTES + o, &maps.go, own_full, x, own0, tma_h, tma_b);
            if constexpr (HAS_GT) {
              tma_load_4d(sOwn + C::SLOT_TQ * C::OWN_BYTES + o, &maps.tq, own_full, x, own0, tma_h, tma_b);
              tma_load_4d(sOwn + C::SLOT_G * C::OWN_BYTES + o, &maps.g, own_full, x, own0, tma_h, tma_b);
            }
          }
        }
      }
      for (int it = 0; it < n_tiles; ++it) {
        const int st = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!mbar_wait(loop_empty + st, ph ^ 1, ab, kAbortBwdLoopEmpty)) break;
        const int l0 = loop_begin + it * BL;
        if (lane == 0) {
          unsigned char* base = sLoop + st * (C::N_LOOP * C::LOOP_BYTES);
          mbar_expect_tx(loop_full + st, C::N_LOOP * C::LOOP_BYTES);
          for (int hf = 0; hf < HALVES; ++hf) {
            const int x = hf * 64, o = hf * (BL * 128);
            if constexpr (OWN_KEYS) {
              tma_load_4d(base + C::SLOT_Q * C::LOOP_BYTES + o, &maps.q, loop_full + st, x, l0, tma_h, tma_b);
              if constexpr (HAS_GO) tma_load_4d(base + C::SLOT_GO * C::LOOP_BYTES + o, &maps.go, loop_full + st, x, l0, tma_h, tma_b);
              if constexpr (HAS_GT) {
                tma_load_4d(base + C::SLOT_TQ * C::LOOP_BYTES + o, &maps.tq, loop_full + st, x, l0, tma_h, tma_b);
                tma_load_4d(base + C::SLOT_G * C::LOOP_BYTES + o, &maps.g, loop_full + st, x, l0, tma_h, tma_b);
              }
            } else {
              tma_load_4d(base + C::SLOT_K * C::LOOP_BYTES + o, &maps.k, loop_full + st, x, l0, tma_h, tma_b);
              tma_load_4d(base + C::SLOT_V * C::LOOP_BYTES + o, &maps.v, loop_full + st, x, l0, tma_h, tma_b);
              if constexpr (HAS_GT) {
                tma_load_4d(base + C::SLOT_TK * C::LOOP_BYTES + o, &maps.tk, loop_full + st, x, l0, tma_h, tma_b);
                tma_load_4d(base + C::SLOT_TV * C::LOOP_BYTES + o, &maps.tv, loop_full + st, x, l0, tma_h, tma_b);
              }
            }
          }
        }
        if constexpr (OWN_KEYS) {
          // per-query statistics of this tile, combined once for all 128 key rows; fetched after the tile
          // loads have been issued, so that the two latencies overlap
          for (int c = lane; c < BL; c += 32) {
            const int i = l0 + c;
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
            sStat[st * BL + c] = s4;
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(loop_full + st);  // second arrival: the statistics are in place
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idesc_sc = make_idesc(Fmt<T>::kIdesc, OWN, BL, 0, 0);  // 128 x 64 scores
      constexpr uint32_t idesc_out = make_idesc(Fmt<T>::kIdesc, OWN, D, 0, 1);  // 128 x D outputs
      auto kdesc = [](uint32_t base, int rows, int ks) {
        return make_smem_desc(base + (ks >> 2) * (rows * 128) + (ks & 3) * 32, 16, 1024);
      };
      auto mndesc = [](uint32_t base, int kk) { return make_smem_desc(base + kk * 2048, BL * 128, 1024); };
      const uint32_t own_base = smem_u32(sOwn);
      auto own_tile = [&](int slot) { return own_base + slot * C::OWN_BYTES; };
      auto score = [&](uint32_t col, uint32_t a_tile, uint32_t b_tile, bool first) {
#pragma unroll
        for (int ks = 0; ks < KSTEPS_D; ++ks)
          umma_ss(tmem + col, kdesc(a_tile, OWN, ks), kdesc(b_tile, BL, ks), idesc_sc, (!first || ks > 0));
      };
      auto outer = [&](uint32_t out_col, uint32_t a_col, uint32_t b_tile, bool accumulate) {
#pragma unroll
        for (int kk = 0; kk < KSTEPS_L; ++kk)
          umma_ts(tmem + out_col, tmem + a_col + kk * 8, mndesc(b_tile, kk), idesc_out, (accumulate || kk > 0));
      };
      bool ok = mbar_wait(own_full, 0, ab, kAbortBwdOwn);
      for (int it = 0; ok && it < n_tiles; ++it) {
        const int st = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!mbar_wait(loop_full + st, ph, ab, kAbortBwdLoopFull)) break;
        tc_fence_after();
        const uint32_t lp = smem_u32(sLoop + st * (C::N_LOOP * C::LOOP_BYTES));
        auto loop_tile = [&](int slot) { return lp + slot * C::LOOP_BYTES; };
        if constexpr (OWN_KEYS) {
          score(C::COL_S, own_tile(C::SLOT_K), loop_tile(C::SLOT_Q), true);
          if constexpr (HAS_GT) {
            score(C::COL_TS, own_tile(C::SLOT_K), loop_tile(C::SLOT_TQ), true);
            score(C::COL_TS, own_tile(C::SLOT_TK), loop_tile(C::SLOT_Q), false);
            score(C::COL_E, own_tile(C::SLOT_V), loop_tile(C::SLOT_G), true);
            score(C::COL_FP, own_tile(C::SLOT_TV), loop_tile(C::SLOT_G), true);
            if constexpr (HAS_GO) score(C::COL_FP, own_tile(C::SLOT_V), loop_tile(C::SLOT_GO), false);
          } else {
            score(C::COL_FP, own_tile(C::SLOT_V), loop_tile(C::SLOT_GO), true);
          }
        } else {
          score(C::COL_S, own_tile(C::SLOT_Q), loop_tile(C::SLOT_K), true);
          if constexpr (HAS_GT) {
            score(C::COL_TS, own_tile(C::SLOT_TQ), loop_tile(C::SLOT_K), true);
            score(C::COL_TS, own_tile(C::SLOT_Q), loop_tile(C::SLOT_TK), false);
            score(C::COL_E, own_tile(C::SLOT_G), loop_tile(C::SLOT_V), true);
            score(C::COL_FP, own_tile(C::SLOT_G), loop_tile(C::SLOT_TV), true);
            if constexpr (HAS_GO) score(C::COL_FP, own_tile(C::SLOT_GO), loop_tile(C::SLOT_V), false);
          } else {
            score(C::COL_FP, own_tile(C::SLOT_GO), loop_tile(C::SLOT_V), true);
          }
        }
        tc_commit(s_full);
        if (!mbar_wait(p_full, it & 1, ab, kAbortBwdPFull)) break;
        tc_fence_after();
        const bool acc = it > 0;
        if constexpr (OWN_KEYS) {
          // dK (OUT0) += gS^T Q + gtS^T tQ ; dV (OUT1) += P^T gO + A^T G
          outer(C::COL_OUT0, C::COL_FP, loop_tile(C::SLOT_Q), acc);
          if constexpr (HAS_GT) {
            outer(C::COL_OUT0, C::COL_E, loop_tile(C::SLOT_TQ), true);
            outer(C::COL_OUT1, C::COL_TS, loop_tile(C::SLOT_G), acc);
            if constexpr (HAS_GO) outer(C::COL_OUT1, C::COL_S, loop_tile(C::SLOT_GO), true);
          } else {
            outer(C::COL_OUT1, C::COL_S, loop_tile(C::SLOT_GO), acc);
          }
        } else {
          // dQ (OUT0) += gS K + gtS tK
          outer(C::COL_OUT0, C::COL_FP, loop_tile(C::SLOT_K), acc);
          if constexpr (HAS_GT) outer(C::COL_OUT0, C::COL_E, loop_tile(C::SLOT_TK), true);
        }
        tc_commit(loop_empty + st);
      }
      tc_commit(done);
    }
  } else {
    // ------------------------------------------------------------------ elementwise + epilogue
    const int quarter = warp & 3;
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

    constexpr int MESZ = MK == 1 ? 1 : 2;  // bytes per mask element
    const unsigned char* mbase = nullptr;
    long long mpitch = 0;
    if constexpr (MK != 0) {
      mbase = reinterpret_cast<const unsigned char*>(a.mask.ptr) +
              ((long long)tma_b * a.mask.stride[0] + (long long)tma_h * a.mask.stride[1]) * MESZ;
      mpitch = a.mask.stride[2] * MESZ;
    }

    for (int it = 0; it < n_tiles; ++it) {
      const int st = it % STAGES;
      const int l0 = loop_begin + it * BL;
      if constexpr (OWN_KEYS) {
        if (!mbar_wait(loop_full + st, (it / STAGES) & 1, ab, kAbortBwdLoopFull)) {
          alive = false;
          break;
        }
      }
      if (!mbar_wait(s_full, it & 1, ab, kAbortBwdSFull)) {
        alive = false;
        break;
      }
      tc_fence_after();
      // does any element of this tile need the mask test?
      bool partial;
      if constexpr (OWN_KEYS) {
        partial = (own0 + OWN > n_valid) || (causal && own0 + OWN - 1 > l0);
      } else {
        partial = (l0 + BL > n_valid) || (causal && l0 + BL - 1 > own0);
      }
      const float4* stat = sStat + st * BL;
#pragma unroll 1
      for (int c = 0; c < BL / 16; ++c) {
        uint32_t s[16], fp[16];
        uint32_t ts[HAS_GT ? 16 : 1], e[HAS_GT ? 16 : 1];
        // MK != 0: the chunk's 16 mask / bias elements, one per column (indices clamped into the tensor;
        // what lies outside is switched off by the index tests below)
        uint32_t mraw[MK == 0 ? 1 : 16];
        if constexpr (MK != 0) {
          if constexpr (OWN_KEYS) {
            const unsigned char* p = mbase + (long long)min(own_idx, L - 1) * MESZ;
#pragma unroll
            for (int x = 0; x < 16; ++x) {
              const unsigned char* el = p + (long long)min(l0 + 16 * c + x, L - 1) * mpitch;
              mraw[x] = MK == 1 ? ldg_nc_u8(el) : ldg_nc_u16(el);
            }
          } else {
            const unsigned char* p = mbase + (long long)min(own_idx, L - 1) * mpitch + (size_t)(l0 + 16 * c) * MESZ;
            uint32_t w[4 * MESZ];
#pragma unroll
            for (int j = 0; j < MESZ; ++j) {
              uint4 r = make_uint4(0u, 0u, 0u, 0u);
              if (l0 + 16 * c + (j + 1) * (16 / MESZ) <= L) r = ldg_nc_v4(p + 16 * j);
              w[4 * j] = r.x, w[4 * j + 1] = r.y, w[4 * j + 2] = r.z, w[4 * j + 3] = r.w;
            }
#pragma unroll
            for (int x = 0; x < 16; ++x)
              mraw[x] = MK == 1 ? ((w[x >> 2] >> ((x & 3) * 8)) & 0xffu) : ((w[x >> 1] >> ((x & 1) * 16)) & 0xffffu);
          }
        }
        tmem_ld16(tbase + C::COL_S + 16 * c, s);
        tmem_ld16(tbase + C::COL_FP + 16 * c, fp);
        if constexpr (HAS_GT) {
          tmem_ld16(tbase + C::COL_TS + 16 * c, ts);
          tmem_ld16(tbase + C::COL_E + 16 * c, e);
        }
        tmem_wait_ld();
        float pv[16], gs[16];
        float av[HAS_GT ? 16 : 1], gt[HAS_GT ? 16 : 1];
#pragma unroll
        for (int x = 0; x < 16; ++x) {
          const int col = 16 * c + x;
          float lse, mu, eps, sub;
          int i, j;
          if constexpr (OWN_KEYS) {
            const float4 s4 = stat[col];
            lse = s4.x, mu = s4.y, eps = s4.z, sub = s4.w;
            i = l0 + col;
            j = own_idx;
          } else {
            lse = r_lse, mu = r_mu, eps = r_eps, sub = r_sub;
            i = own_idx;
            j = l0 + col;
          }
          float arg = __uint_as_float(s[x]) * scale_log2 - lse;
          if constexpr (MK == 2) arg = fmaf(unpack1<T>(mraw[x]), kLog2e, arg);  // scores are in log2 units
          float p = fast_exp2(arg);
          if constexpr (MK == 1)
            if (mraw[x] == 0u) p = 0.f;
          if (partial && (j >= n_valid || (causal && j > i))) p = 0.f;
          pv[x] = p;
          if constexpr (HAS_GT) {
            const float tm = __uint_as_float(ts[x]) * a.sm_scale - mu;
            const float eb = __uint_as_float(e[x]) - eps;
            av[x] = p * tm;
            gt[x] = p * eb;
            gs[x] = p * (eb * tm + __uint_as_float(fp[x]) - sub);
          } else {
            gs[x] = p * (__uint_as_float(fp[x]) - sub);
          }
        }
        uint32_t pk[8];
#pragma unroll
        for (int x = 0; x < 8; ++x) pk[x] = Elem<T>::pack(gs[2 * x], gs[2 * x + 1]);
        tmem_st8(tbase + C::COL_FP + 8 * c, pk);
        if constexpr (HAS_GT) {
#pragma unroll
          for (int x = 0; x < 8; ++x) pk[x] = Elem<T>::pack(gt[2 * x], gt[2 * x + 1]);
          tmem_st8(tbase + C::COL_E + 8 * c, pk);
          if constexpr (OWN_KEYS) {
#pragma unroll
            for (int x = 0; x < 8; ++x) pk[x] = Elem<T>::pack(av[2 * x], av[2 * x + 1]);
            tmem_st8(tbase + C::COL_TS + 8 * c, pk);
          }
        }
        if constexpr (OWN_KEYS && HAS_GO) {
#pragma unroll
          for (int x = 0; x < 8; ++x) pk[x] = Elem<T>::pack(pv[2 * x], pv[2 * x + 1]);
          tmem_st8(tbase + C::COL_S + 8 * c, pk);
        }
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(p_full);
    }

    // ---- epilogue ----
    if (alive && n_tiles > 0) alive = mbar_wait(done, 0, ab, kAbortBwdDone);
    if (alive) {
      tc_fence_after();
      const bool in_range = own_idx < L;
      auto store_rows = [&](void* gptr, uint32_t col0, float mul) {
        T* g = reinterpret_cast<T*>(gptr) + ((size_t)bh * L + own_idx) * D;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
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
template <typename T, int D, bool OWN_KEYS, bool HAS_GO, bool HAS_GT, int MK>
static int launch_half(const jvpfa_bwd_args& a, cudaStream_t stream, int* status, bool overlap_previous) {
  static_assert(MK >= 0 && MK <= 2, "mask mode");
  using C = BwdCfg<D, OWN_KEYS, HAS_GO, HAS_GT>;
  BwdMaps m;
  const long long BH = (long long)a.B * a.H;
  const CUtensorMapDataType dt = Fmt<T>::kTma;
  const int key_rows = OWN_KEYS ? C::OWN : C::BL;
  const int qry_rows = OWN_KEYS ? C::BL : C::OWN;
  bool ok = encode_map4d(&m.k, dt, a.k, D, a.L, a.H, a.B, a.in_stride, key_rows) && encode_map4d(&m.v, dt, a.v, D, a.L, a.H, a.B, a.in_stride, key_rows) &&
            encode_map4d(&m.q, dt, a.q, D, a.L, a.H, a.B, a.in_stride, qry_rows);
  m.tk = m.tv = m.k;
  m.go = m.tq = m.g = m.q;
  if (HAS_GO) ok = ok && encode_map4d(&m.go, dt, a.go, D, a.L, a.H, a.B, nullptr, qry_rows);
  if (HAS_GT)
    ok = ok && encode_map4d(&m.tk, dt, a.tk, D, a.L, a.H, a.B, a.in_stride, key_rows) && encode_map4d(&m.tv, dt, a.tv, D, a.L, a.H, a.B, a.in_stride, key_rows) &&
         encode_map4d(&m.tq, dt, a.tq, D, a.L, a.H, a.B, a.in_stride, qry_rows) && encode_map4d(&m.g, dt, a.gto, D, a.L, a.H, a.B, nullptr, qry_rows);
  if (!ok) {
    set_last_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled(bwd)");
    return JVPFA_ERR_CUDA;
  }
  auto kern = bwd_tc5_kernel<T, D, OWN_KEYS, HAS_GO, HAS_GT, MK>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
  if (e != cudaSuccess) {
    set_last_cuda_error(e, "cudaFuncSetAttribute(bwd_tc5)");
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
    set_last_cuda_error(e, "launch bwd_tc5");
    return JVPFA_ERR_CUDA;
  }
  return JVPFA_OK;
}

template <typename T, int D, bool HAS_GO, bool HAS_GT, int MK>
static int launch_both(const jvpfa_bwd_args& a, cudaStream_t s) {
  int* status = tc5_status_device_ptr();
  if (!status) {
    set_last_cuda_error(cudaErrorUnknown, "status word address");
    return JVPFA_ERR_CUDA;
  }
  int rc = JVPFA_OK;
  rc = launch_half<T, D, true, HAS_GO, HAS_GT, MK>(a, s, status, false);
  if (rc) return rc;
  rc = launch_half<T, D, false, HAS_GO, HAS_GT, MK>(a, s, status, true);
  return rc;
}

template <typename T, int D, int MK>
static int launch_d(const jvpfa_bwd_args& a, cudaStream_t s) {
  const bool go = a.go != nullptr, gt = a.gto != nullptr;
  if (go && gt) return launch_both<T, D, true, true, MK>(a, s);
  if (gt) return launch_both<T, D, false, true, MK>(a, s);
  return launch_both<T, D, true, false, MK>(a, s);
}

template <typename T>
static int launch_t(const jvpfa_bwd_args& a, cudaStream_t s) {
  if (a.D != 128) return JVPFA_ERR_UNSUPPORTED;  // D = 64 has its own kernels (bwd_tc5_d64.cu)
  if (a.mask.kind == JVPFA_MASK_BOOL) return launch_d<T, 128, 1>(a, s);
  if (a.mask.kind == JVPFA_MASK_BIAS) return launch_d<T, 128, 2>(a, s);
  return launch_d<T, 128, 0>(a, s);
}

}  // namespace tc5

bool bwd_tc5_eligible(const jvpfa_bwd_args& a) {
  if (a.dtype != JVPFA_BF16 && a.dtype != JVPFA_FP16) return false;
  if (a.D != 64 && a.D != 128) return false;
  const int k = a.mask.kind;
  if (k == JVPFA_MASK_NONE || k == JVPFA_MASK_CAUSAL || k == JVPFA_MASK_KVLEN) return true;
  // Boolean masks and bias: the elementwise threads read 16-byte pieces of mask rows
  if ((a.L & 15) != 0) return false;
  if (k == JVPFA_MASK_BIAS && a.mask.bias_dtype != a.dtype) return false;
  const long long esz = k == JVPFA_MASK_BOOL ? 1 : 2;
  if (a.mask.stride[3] != 1 || (reinterpret_cast<uintptr_t>(a.mask.ptr) & 15u) != 0) return false;
  for (int d = 0; d < 3; ++d)
    if (a.mask.stride[d] < 0 || ((a.mask.stride[d] * esz) & 15) != 0) return false;
  return true;
}

int launch_bwd_tc5(const jvpfa_bwd_args& a, cudaStream_t s) {
  if (a.D == 64) {
    // one pass over the score tiles when the caller gave the dQ accumulation buffer (bwd_tc5_fused64.cu)
    if (bwd_tc5_fused64_eligible(a)) return launch_bwd_tc5_fused64(a, s);
    return launch_bwd_tc5_d64(a, s);  // two pipelined launches (bwd_tc5_d64.cu)
  }
  // Head dimension 128 without a user mask or bias: the pipelined kernels of bwd_tc5_pipe128.cu
  if (bwd_tc5_pipe128_eligible(a)) return launch_bwd_tc5_pipe128(a, s);
  return a.dtype == JVPFA_BF16 ? tc5::launch_t<__nv_bfloat16>(a, s) : tc5::launch_t<__half>(a, s);
}

}  // namespace jvpfa
