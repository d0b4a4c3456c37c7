// Shared device helpers for the register-tiled (mma.sync) attention kernels:
// warp-level MMA fragments for bf16 / fp16 (m16n8k16) and fp32 (m16n8k8 TF32 issued
// three times on a hi/lo split, "3xTF32"), cp.async tile staging, and the mask /
// bias accessor used inside every tile loop.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/jvpfa.h"

namespace jvpfa {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// ----------------------------------------------------------------------------------------------
// Element traits
// ----------------------------------------------------------------------------------------------
template <typename T>
struct Elem;

template <>
struct Elem<__nv_bfloat16> {
  static constexpr bool k16 = true;
  static constexpr int kPad = 8;  // smem row padding in elements (keeps 16-byte rows, spreads banks)
  static constexpr int kKStep = 16;
  __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __device__ static __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
  __device__ static __forceinline__ __nv_bfloat16 from_float(float x) { return __float2bfloat16_rn(x); }
};

template <>
struct Elem<__half> {
  static constexpr bool k16 = true;
  static constexpr int kPad = 8;
  static constexpr int kKStep = 16;
  __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __device__ static __forceinline__ float to_float(__half x) { return __half2float(x); }
  __device__ static __forceinline__ __half from_float(float x) { return __float2half_rn(x); }
};

template <>
struct Elem<float> {
  static constexpr bool k16 = false;
  static constexpr bool kSplit = true;  // every product is three TF32 MMAs on a hi/lo split
  static constexpr int kPad = 4;
  static constexpr int kKStep = 8;
  __device__ static __forceinline__ float to_float(float x) { return x; }
  __device__ static __forceinline__ float from_float(float x) { return x; }
};

// fp32 in memory, products as one TF32 MMA (JVPFA_FP32_TF32): the precision of upstream's fp32 path, whose
// tl.dot calls run on TF32 tensor cores (jvp_attention.py:233-236, 314-322).  Relative error about 5e-4.
struct tf32x1 {
  float v;
};
template <>
struct Elem<tf32x1> {
  static constexpr bool k16 = false;
  static constexpr bool kSplit = false;
  static constexpr int kPad = 4;
  static constexpr int kKStep = 8;
  __device__ static __forceinline__ float to_float(tf32x1 x) { return x.v; }
  __device__ static __forceinline__ tf32x1 from_float(float x) { return tf32x1{x}; }
};

// ----------------------------------------------------------------------------------------------
// Raw MMA instructions.  Lane decomposition used everywhere: g = lane >> 2 (0..7), t = lane & 3.
//   C (16x8 fp32): c0=(g,2t) c1=(g,2t+1) c2=(g+8,2t) c3=(g+8,2t+1)
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_16816(const __nv_bfloat16*, float c[4], const uint32_t a[4],
                                          const uint32_t b[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void mma_16816(const __half*, float c[4], const uint32_t a[4],
                                          const uint32_t b[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void mma_1688_tf32(float c[4], const uint32_t a[4], const uint32_t b[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// Split an fp32 value into a TF32 "hi" part and the TF32 rounding of the remainder.
__device__ __forceinline__ void split_tf32(float x, uint32_t& hi, uint32_t& lo) {
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hi) : "f"(x));
  float r = x - __uint_as_float(hi);
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lo) : "f"(r));
}
// The same for element type T: types that multiply in one pass have no lo part.
template <typename T>
__device__ __forceinline__ void split_t(float x, uint32_t& hi, uint32_t& lo) {
  if constexpr (Elem<T>::kSplit) {
    split_tf32(x, hi, lo);
  } else {
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hi) : "f"(x));
    lo = 0u;
  }
}

// ----------------------------------------------------------------------------------------------
// Fragments.  For 16-bit types a fragment is the packed register set of m16n8k16; for fp32 it
// carries the hi and lo TF32 halves so that one logical MMA is lo*hi + hi*lo + hi*hi.
// ----------------------------------------------------------------------------------------------
template <typename T, bool k16 = Elem<T>::k16>
struct FragA;
template <typename T, bool k16 = Elem<T>::k16>
struct FragB;

template <typename T>
struct FragA<T, true> {
  uint32_t r[4];
};
template <typename T>
struct FragB<T, true> {
  uint32_t r[2];
};
template <typename T>
struct FragA<T, false> {
  uint32_t hi[4], lo[4];
};
template <typename T>
struct FragB<T, false> {
  uint32_t hi[2], lo[2];
};

template <typename T>
__device__ __forceinline__ void mma(float c[4], const FragA<T, true>& a, const FragB<T, true>& b) {
  mma_16816(static_cast<const T*>(nullptr), c, a.r, b.r);
}
template <typename T>
__device__ __forceinline__ void mma(float c[4], const FragA<T, false>& a, const FragB<T, false>& b) {
  if constexpr (Elem<T>::kSplit) {
    mma_1688_tf32(c, a.lo, b.hi);
    mma_1688_tf32(c, a.hi, b.lo);
  }
  mma_1688_tf32(c, a.hi, b.hi);
}

// A fragment from a row-major smem tile s[row][k] (k contiguous, leading dimension ld elements):
// rows r0..r0+15, contraction slice k0..k0+KStep-1.
template <typename T>
__device__ __forceinline__ void load_a(FragA<T, true>& f, const T* s, int ld, int r0, int k0, int lane) {
  const int g = lane >> 2, t = lane & 3;
  const T* p0 = s + (r0 + g) * ld + k0 + 2 * t;
  const T* p1 = p0 + 8 * ld;
  f.r[0] = *reinterpret_cast<const uint32_t*>(p0);
  f.r[1] = *reinterpret_cast<const uint32_t*>(p1);
  f.r[2] = *reinterpret_cast<const uint32_t*>(p0 + 8);
  f.r[3] = *reinterpret_cast<const uint32_t*>(p1 + 8);
}
template <typename T>
__device__ __forceinline__ void load_a(FragA<T, false>& f, const T* s, int ld, int r0, int k0, int lane) {
  const int g = lane >> 2, t = lane & 3;
  const float* p0 = reinterpret_cast<const float*>(s) + (r0 + g) * ld + k0 + t;
  const float* p1 = p0 + 8 * ld;
  split_t<T>(p0[0], f.hi[0], f.lo[0]);
  split_t<T>(p1[0], f.hi[1], f.lo[1]);
  split_t<T>(p0[4], f.hi[2], f.lo[2]);
  split_t<T>(p1[4], f.hi[3], f.lo[3]);
}

// B fragment, "NT": the smem tile is s[n][k] with k contiguous (C = A * s^T).
template <typename T>
__device__ __forceinline__ void load_b_nt(FragB<T, true>& f, const T* s, int ld, int n0, int k0, int lane) {
  const int g = lane >> 2, t = lane & 3;
  const T* p = s + (n0 + g) * ld + k0 + 2 * t;
  f.r[0] = *reinterpret_cast<const uint32_t*>(p);
  f.r[1] = *reinterpret_cast<const uint32_t*>(p + 8);
}
template <typename T>
__device__ __forceinline__ void load_b_nt(FragB<T, false>& f, const T* s, int ld, int n0, int k0, int lane) {
  const int g = lane >> 2, t = lane & 3;
  const float* p = reinterpret_cast<const float*>(s) + (n0 + g) * ld + k0 + t;
  split_t<T>(p[0], f.hi[0], f.lo[0]);
  split_t<T>(p[4], f.hi[1], f.lo[1]);
}

// B fragment, "NN": the smem tile is s[k][n] with n contiguous (C = A * s).
// 16-bit: slot pairs (2t,2t+1) and (2t+8,2t+9) are two consecutive rows of s.
// fp32: the A operand of these products comes straight from an accumulator tile whose
// columns (2t, 2t+1) sit in MMA k-slots (t, t+4) (see a_from_acc); the same permutation
// of the contraction index is applied here, so slot t reads row k0+2t and slot t+4 reads
// row k0+2t+1.
template <typename T>
__device__ __forceinline__ void load_b_nn(FragB<T, true>& f, const T* s, int ld, int k0, int n0, int lane) {
  const int g = lane >> 2, t = lane & 3;
  const unsigned short* p = reinterpret_cast<const unsigned short*>(s) + (k0 + 2 * t) * ld + n0 + g;
  f.r[0] = (uint32_t)p[0] | ((uint32_t)p[ld] << 16);
  f.r[1] = (uint32_t)p[8 * ld] | ((uint32_t)p[9 * ld] << 16);
}
template <typename T>
__device__ __forceinline__ void load_b_nn(FragB<T, false>& f, const T* s, int ld, int k0, int n0, int lane) {
  const int g = lane >> 2, t = lane & 3;
  const float* p = reinterpret_cast<const float*>(s) + (k0 + 2 * t) * ld + n0 + g;
  split_t<T>(p[0], f.hi[0], f.lo[0]);
  split_t<T>(p[ld], f.hi[1], f.lo[1]);
}

// A fragment taken from an accumulator-layout tile acc[n_tile][4] (16 rows x 8*n_tiles cols),
// contraction step kk (KStep columns starting at kk*KStep).
template <typename T>
__device__ __forceinline__ void a_from_acc(FragA<T, true>& f, const float (*acc)[4], int kk) {
  const float* c0 = acc[2 * kk];
  const float* c1 = acc[2 * kk + 1];
  f.r[0] = Elem<T>::pack(c0[0], c0[1]);
  f.r[1] = Elem<T>::pack(c0[2], c0[3]);
  f.r[2] = Elem<T>::pack(c1[0], c1[1]);
  f.r[3] = Elem<T>::pack(c1[2], c1[3]);
}
template <typename T>
__device__ __forceinline__ void a_from_acc(FragA<T, false>& f, const float (*acc)[4], int kk) {
  const float* c = acc[kk];
  split_t<T>(c[0], f.hi[0], f.lo[0]);  // slot t    <- column 2t,   row g
  split_t<T>(c[2], f.hi[1], f.lo[1]);  // slot t    <- column 2t,   row g+8
  split_t<T>(c[1], f.hi[2], f.lo[2]);  // slot t+4  <- column 2t+1, row g
  split_t<T>(c[3], f.hi[3], f.lo[3]);  // slot t+4  <- column 2t+1, row g+8
}

// ----------------------------------------------------------------------------------------------
// cp.async staging of a [ROWS][D] tile (rows row0.. of one head) into padded smem.
// Rows at or beyond L are zero-filled.
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, int src_bytes) {
  uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(gsrc), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

// row_stride: elements between consecutive rows of the head in global memory (D for a row-major head; the row stride of
// a strided (batch, head, row) layout otherwise; the row itself is contiguous).
template <typename T, int ROWS, int D, int NTHREADS>
__device__ __forceinline__ void stage_tile(T* s, const T* head, int row0, int L, int tid, long long row_stride = D) {
  constexpr int LD = D + Elem<T>::kPad;
  constexpr int VEC = 16 / (int)sizeof(T);
  constexpr int VPR = D / VEC;
  for (int idx = tid; idx < ROWS * VPR; idx += NTHREADS) {
    const int r = idx / VPR;
    const int c = (idx - r * VPR) * VEC;
    const int gr = row0 + r;
    const bool ok = gr < L;
    cp_async16(s + r * LD + c, head + (long long)(ok ? gr : 0) * row_stride + c, ok ? 16 : 0);
  }
}

// ----------------------------------------------------------------------------------------------
// Mask / bias accessor for one (batch, head).
// ----------------------------------------------------------------------------------------------
struct MaskView {
  int kind;
  int L;
  int kv_len;         // KVLEN: valid keys of this batch entry
  int bias_dtype;     // BIAS: jvpfa_dtype
  const void* base;   // BOOL / BIAS: pointer already offset to (b, h, 0, 0)
  long long si, sj;   // element strides along query / key

  __device__ __forceinline__ bool allowed(int i, int j) const {
    if (i >= L || j >= L) return false;
    switch (kind) {
      case JVPFA_MASK_CAUSAL:
        return j <= i;
      case JVPFA_MASK_KVLEN:
        return j < kv_len;
      case JVPFA_MASK_BOOL:
        return reinterpret_cast<const uint8_t*>(base)[i * si + j * sj] != 0;
      default:
        return true;
    }
  }
  // allowed() and bias() for the two neighbouring keys j, j + 1 (j even) of query i at once.  When the key
  // stride is 1 and the address allows it, the two mask bytes / bias elements come from one load.
  __device__ __forceinline__ void pair(int i, int j, bool ok[2], float b[2]) const {
    b[0] = b[1] = 0.f;
    if ((kind == JVPFA_MASK_BOOL || kind == JVPFA_MASK_BIAS) && sj == 1 && i < L && j + 1 < L) {
      const long long off = i * si + j;
      if (kind == JVPFA_MASK_BOOL) {
        const uint8_t* p = reinterpret_cast<const uint8_t*>(base) + off;
        if ((reinterpret_cast<uintptr_t>(p) & 1u) == 0) {
          const uint32_t w = *reinterpret_cast<const uint16_t*>(p);
          ok[0] = (w & 0xffu) != 0, ok[1] = (w >> 8) != 0;
          return;
        }
      } else if (bias_dtype == JVPFA_FP32) {
        const float* p = reinterpret_cast<const float*>(base) + off;
        if ((reinterpret_cast<uintptr_t>(p) & 7u) == 0) {
          const float2 v = *reinterpret_cast<const float2*>(p);
          ok[0] = ok[1] = true, b[0] = v.x, b[1] = v.y;
          return;
        }
      } else {
        const uint16_t* p = reinterpret_cast<const uint16_t*>(base) + off;
        if ((reinterpret_cast<uintptr_t>(p) & 3u) == 0) {
          const uint32_t w = *reinterpret_cast<const uint32_t*>(p);
          ok[0] = ok[1] = true;
          if (bias_dtype == JVPFA_BF16) {
            b[0] = __uint_as_float(w << 16), b[1] = __uint_as_float(w & 0xffff0000u);
          } else {
            const float2 v = __half22float2(*reinterpret_cast<const __half2*>(&w));
            b[0] = v.x, b[1] = v.y;
          }
          return;
        }
      }
    }
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      ok[e] = allowed(i, j + e);
      if (ok[e]) b[e] = bias(i, j + e);
    }
  }
  // Additive bias in natural units (0 unless kind == BIAS).  Only call for in-range (i, j).
  __device__ __forceinline__ float bias(int i, int j) const {
    if (kind != JVPFA_MASK_BIAS) return 0.f;
    const long long off = i * si + j * sj;
    if (bias_dtype == JVPFA_FP32) return reinterpret_cast<const float*>(base)[off];
    if (bias_dtype == JVPFA_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[off]);
    return __half2float(reinterpret_cast<const __half*>(base)[off]);
  }
};

__device__ __forceinline__ MaskView make_mask_view(const jvpfa_mask& m, int b, int h, int L) {
  MaskView v;
  v.kind = m.kind;
  v.L = L;
  v.kv_len = L;
  v.bias_dtype = m.bias_dtype;
  v.base = nullptr;
  v.si = m.stride[2];
  v.sj = m.stride[3];
  if (m.kind == JVPFA_MASK_KVLEN) {
    int n = m.kv_len[b];
    v.kv_len = n < 0 ? 0 : (n > L ? L : n);
  } else if (m.kind == JVPFA_MASK_BOOL) {
    v.base = reinterpret_cast<const uint8_t*>(m.ptr) + (long long)b * m.stride[0] + (long long)h * m.stride[1];
  } else if (m.kind == JVPFA_MASK_BIAS) {
    const long long off = (long long)b * m.stride[0] + (long long)h * m.stride[1];
    const int esz = (m.bias_dtype == JVPFA_FP32) ? 4 : 2;
    v.base = reinterpret_cast<const uint8_t*>(m.ptr) + off * esz;
  }
  return v;
}

// Reductions across the four lanes that share an accumulator row.
__device__ __forceinline__ float quad_max(float x) {
  x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 1));
  x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 2));
  return x;
}
__device__ __forceinline__ float quad_sum(float x) {
  x += __shfl_xor_sync(0xffffffffu, x, 1);
  x += __shfl_xor_sync(0xffffffffu, x, 2);
  return x;
}

// Host-side launch helpers implemented by each kernel translation unit.
int launch_fwd_generic(const jvpfa_fwd_args& a, cudaStream_t stream);
int launch_pre(const jvpfa_pre_args& a, cudaStream_t stream);
int launch_bwd_generic(const jvpfa_bwd_args& a, cudaStream_t stream);
int launch_mask_check(const jvpfa_mask_check_args& a, cudaStream_t stream);
int launch_mask_tiles(const jvpfa_mask_tiles_args& a, cudaStream_t stream);
int launch_fwd_tc5(const jvpfa_fwd_args& a, cudaStream_t stream);
bool fwd_tc5_eligible(const jvpfa_fwd_args& a);
int tc5_read_status(int* out, int clear);
int tc5_status_peek();
int tc5_inject_status(int code);
int* tc5_status_device_ptr();
int launch_bwd_tc5(const jvpfa_bwd_args& a, cudaStream_t stream);
int launch_bwd_tc5_d64(const jvpfa_bwd_args& a, cudaStream_t stream);
int launch_bwd_tc5_fused64(const jvpfa_bwd_args& a, cudaStream_t stream);
bool bwd_tc5_fused64_eligible(const jvpfa_bwd_args& a);
int launch_fwd_tc5_pair64(const jvpfa_fwd_args& a, cudaStream_t stream);
int launch_fwd_tc5_pipe128(const jvpfa_fwd_args& a, cudaStream_t stream);
bool bwd_tc5_pipe128_eligible(const jvpfa_bwd_args& a);
int launch_bwd_tc5_pipe128(const jvpfa_bwd_args& a, cudaStream_t stream);
bool bwd_tc5_eligible(const jvpfa_bwd_args& a);
void set_last_cuda_error(cudaError_t e, const char* where);
int check_pre_request(const jvpfa_pre_args* a);
int check_bwd_request(const jvpfa_bwd_args* a);

}  // namespace jvpfa
