// One pass over a user mask that answers what upstream asks of it before a forward
// (jvp_flash_attention/jvp_attention.py:2438-2457): does every head of a boolean mask keep at least
// one entry, does a floating-point mask contain inf or NaN, does every head of it have at least one
// entry other than the masking constant -100.  Upstream answers with four eager reductions over the
// whole mask and a host synchronisation after each; here one HBM-bound kernel writes one int32 per
// head plus one "bad value" word, which the caller reads back once.
//
// Work split: blockIdx.y = head of the mask (its own batch x head extents: broadcast dimensions
// count once), blockIdx.x = a slice of that head's rows.  A row is read as 16-byte vectors when its
// key stride is 1 and it starts on a 16-byte boundary, element by element otherwise.
#include "common.cuh"

namespace jvpfa {

namespace {

constexpr int kCheckThreads = 256;

// bit 0: the element counts as "live" (true / not the masking constant -100); bit 1: inf; bit 2: NaN
__device__ __forceinline__ uint32_t classify_bits(uint32_t x, uint32_t mask_const, uint32_t exp_mask, uint32_t man_mask) {
  uint32_t r = x != mask_const ? 1u : 0u;
  if ((x & exp_mask) == exp_mask) r |= (x & man_mask) ? 4u : 2u;
  return r;
}
template <int KIND_DTYPE>
__device__ __forceinline__ uint32_t classify16(uint32_t h) {
  if constexpr (KIND_DTYPE == JVPFA_BF16)
    return classify_bits(h & 0xffffu, 0xC2C8u, 0x7f80u, 0x007fu);
  else
    return classify_bits(h & 0xffffu, 0xD640u, 0x7c00u, 0x03ffu);
}
__device__ __forceinline__ uint32_t classify32(uint32_t w) { return classify_bits(w, 0xC2C80000u, 0x7f800000u, 0x007fffffu); }

// MODE 0: uint8 mask; 1: bf16; 2: fp16; 3: fp32
template <int MODE>
__device__ __forceinline__ uint32_t classify_word(uint32_t w) {
  if constexpr (MODE == 0) return w != 0u ? 1u : 0u;
  if constexpr (MODE == 1) return classify16<JVPFA_BF16>(w) | classify16<JVPFA_BF16>(w >> 16);
  if constexpr (MODE == 2) return classify16<JVPFA_FP16>(w) | classify16<JVPFA_FP16>(w >> 16);
  return classify32(w);
}

template <int MODE>
__device__ __forceinline__ uint32_t classify_elem(const unsigned char* p) {
  if constexpr (MODE == 0) return *p != 0 ? 1u : 0u;
  if constexpr (MODE == 1) return classify16<JVPFA_BF16>(*reinterpret_cast<const uint16_t*>(p));
  if constexpr (MODE == 2) return classify16<JVPFA_FP16>(*reinterpret_cast<const uint16_t*>(p));
  return classify32(*reinterpret_cast<const uint32_t*>(p));
}

template <int MODE>
__global__ void __launch_bounds__(kCheckThreads) mask_check_kernel(const jvpfa_mask m, int n_h, int n_rows, int L,
                                                                   int rows_per_cta, int32_t* out) {
  constexpr int ESZ = MODE == 0 ? 1 : (MODE == 3 ? 4 : 2);
  constexpr int EPV = 16 / ESZ;  // elements per 16-byte vector
  const int head = blockIdx.y;
  const int b = head / n_h, h = head - b * n_h;
  const int r0 = blockIdx.x * rows_per_cta;
  const int r1 = min(n_rows, r0 + rows_per_cta);
  const unsigned char* base =
      reinterpret_cast<const unsigned char*>(m.ptr) + ((long long)b * m.stride[0] + (long long)h * m.stride[1]) * ESZ;
  const long long row_bytes = m.stride[2] * ESZ;
  const bool vec = m.stride[3] == 1 && (L % EPV) == 0 && (reinterpret_cast<uintptr_t>(base) & 15u) == 0 &&
                   (row_bytes & 15) == 0;
  uint32_t acc = 0;
  auto take = [&](const uint4 x) {
    acc |= classify_word<MODE>(x.x) | classify_word<MODE>(x.y) | classify_word<MODE>(x.z) | classify_word<MODE>(x.w);
  };
  if (vec) {
    const int vpr = L / EPV;
    if (row_bytes == (long long)L * ESZ) {  // the slice is one contiguous range
      const uint4* p = reinterpret_cast<const uint4*>(base + (long long)r0 * row_bytes);
      const int total = (r1 - r0) * vpr;
#pragma unroll 8
      for (int idx = threadIdx.x; idx < total; idx += kCheckThreads) take(__ldg(p + idx));
    } else {
      for (int r = r0; r < r1; ++r) {
        const uint4* p = reinterpret_cast<const uint4*>(base + (long long)r * row_bytes);
#pragma unroll 4
        for (int c = threadIdx.x; c < vpr; c += kCheckThreads) take(__ldg(p + c));
      }
    }
  } else {
    for (int r = r0; r < r1; ++r) {
      const unsigned char* p = base + (long long)r * row_bytes;
      for (int c = threadIdx.x; c < L; c += kCheckThreads) acc |= classify_elem<MODE>(p + (long long)c * m.stride[3] * ESZ);
    }
  }
  const int live = __syncthreads_or((int)(acc & 1u));
  const int inf = __syncthreads_or((int)(acc & 2u));
  const int nan = __syncthreads_or((int)(acc & 4u));
  if (threadIdx.x == 0) {
    if (live) out[1 + head] = 1;  // every writer stores the same value
    if (inf || nan) atomicOr(out, (inf ? 1 : 0) | (nan ? 2 : 0));
  }
}

// Tile summary of a boolean mask.  One CTA = one 128-row tile row of one head x eight 64-key tiles
// (512 bytes of each row): lane l of a warp reads bytes [16 l, 16 l + 16) of a row, so four
// neighbouring lanes cover one tile; the eight warps share out the rows.
__global__ void __launch_bounds__(256) mask_tiles_kernel(const jvpfa_mask m, int n_h, int n_rows, int L, int n_qt,
                                                         int n_words, unsigned char* tile_live, int32_t* head_live,
                                                         unsigned long long* tile_live_t, int n_kt128, int n_words_t) {
  __shared__ unsigned int s_bits;
  const int head = blockIdx.z, qt = blockIdx.y, kg = blockIdx.x;  // kg: group of eight key tiles
  const int b = head / n_h, h = head - b * n_h;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned char* base = reinterpret_cast<const unsigned char*>(m.ptr) + (long long)b * m.stride[0] +
                              (long long)h * m.stride[1];
  if (threadIdx.x == 0) s_bits = 0u;
  __syncthreads();
  const int col = kg * 512 + lane * 16;
  const int r0 = qt * 128, r1 = min(n_rows, r0 + 128);
  unsigned int any = 0u;
  if (col + 16 <= L) {
#pragma unroll 4
    for (int r = r0 + warp; r < r1; r += 8) {
      const uint4 x = __ldg(reinterpret_cast<const uint4*>(base + (long long)r * m.stride[2] + col));
      any |= x.x | x.y | x.z | x.w;
    }
  }
  const unsigned int vote = __ballot_sync(0xffffffffu, any != 0u);  // bit l: lane l saw a true entry
  if (lane == 0 && vote != 0u) {
    unsigned int tiles = 0u;
#pragma unroll
    for (int t = 0; t < 8; ++t)
      if (vote & (0xfu << (4 * t))) tiles |= 1u << t;
    atomicOr(&s_bits, tiles);
  }
  __syncthreads();
  if (threadIdx.x == 0 && s_bits != 0u) {
    // byte kg of the entry's words (little endian: byte k of a word holds its bits 8k .. 8k+7)
    tile_live[((long long)head * n_qt + qt) * n_words * 8 + kg] = (unsigned char)s_bits;
    if (head_live) {
      head_live[head] = 1;
      atomicAdd(head_live + gridDim.z, __popc(s_bits));  // live tiles of the whole mask
    }
    if (tile_live_t) {  // the transposed summary: per 128-key tile, one bit per 128-query tile
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if ((s_bits >> (2 * j)) & 3u)
          atomicOr(tile_live_t + ((long long)head * n_kt128 + 4 * kg + j) * n_words_t + (qt >> 6), 1ull << (qt & 63));
    }
  }
}

}  // namespace

int launch_mask_tiles(const jvpfa_mask_tiles_args& a, cudaStream_t stream) {
  const int n_kt = (a.L + 63) / 64;
  const int n_words = (n_kt + 63) / 64;
  const int n_qt = a.n_rows == 1 ? 1 : (a.L + 127) / 128;
  const dim3 grid((unsigned)((n_kt + 7) / 8), (unsigned)n_qt, (unsigned)(a.n_b * a.n_h));
  const int n_kt128 = (a.L + 127) / 128;
  const int n_words_t = (n_qt + 63) / 64;
  mask_tiles_kernel<<<grid, 256, 0, stream>>>(a.mask, a.n_h, a.n_rows, a.L, n_qt, n_words,
                                              reinterpret_cast<unsigned char*>(a.tile_live), a.head_live,
                                              reinterpret_cast<unsigned long long*>(a.tile_live_t), n_kt128, n_words_t);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_cuda_error(e, "launch mask_tiles");
    return JVPFA_ERR_CUDA;
  }
  return JVPFA_OK;
}

int launch_mask_check(const jvpfa_mask_check_args& a, cudaStream_t stream) {
  const int n_heads = a.n_b * a.n_h;
  // about 32 KiB of mask per CTA (eight 16-byte loads per thread), at least one row: a 100 MB mask gives
  // some 3000 CTAs, enough loads in flight to run at HBM speed
  const long long row_bytes = (long long)a.L * (a.mask.kind == JVPFA_MASK_BOOL ? 1 : (a.mask.bias_dtype == JVPFA_FP32 ? 4 : 2));
  long long rpc = (32ll << 10) / row_bytes;
  if (rpc < 1) rpc = 1;
  if (rpc > a.n_rows) rpc = a.n_rows;
  const dim3 grid((unsigned)((a.n_rows + rpc - 1) / rpc), (unsigned)n_heads);
  if (a.mask.kind == JVPFA_MASK_BOOL)
    mask_check_kernel<0><<<grid, kCheckThreads, 0, stream>>>(a.mask, a.n_h, a.n_rows, a.L, (int)rpc, a.out);
  else if (a.mask.bias_dtype == JVPFA_BF16)
    mask_check_kernel<1><<<grid, kCheckThreads, 0, stream>>>(a.mask, a.n_h, a.n_rows, a.L, (int)rpc, a.out);
  else if (a.mask.bias_dtype == JVPFA_FP16)
    mask_check_kernel<2><<<grid, kCheckThreads, 0, stream>>>(a.mask, a.n_h, a.n_rows, a.L, (int)rpc, a.out);
  else
    mask_check_kernel<3><<<grid, kCheckThreads, 0, stream>>>(a.mask, a.n_h, a.n_rows, a.L, (int)rpc, a.out);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_cuda_error(e, "launch mask_check");
    return JVPFA_ERR_CUDA;
  }
  return JVPFA_OK;
}

}  // namespace jvpfa
