// Row norms in their general form, for the places the LayerNorm-with-bias kernel does not cover:
//   layer form   y = (x - mean) / sqrt(mean((x - mean)^2) + eps) * g (+ b)
//   RMS form     y = x / sqrt(mean(x^2) + eps) * g (+ b)
// gain and bias may each be absent.  The source is float or bfloat16 with a free row stride (a
// column range of a wider buffer: a latent beside the queries of one projection) and an optional
// row gather; statistics are two-pass in 32-bit.  Three destinations:
//   rows      dst[r, :] = y                      (float or bfloat16, free row stride)
//   scatter   dst[dst_rows[r], :] = y            (the rows of a paged cache, by slot)
//   add       dst[r, :] += y                     (float: a norm behind a sublayer, summed into the
//                                                 32-bit residual stream)
// In groups: a row is split into `groups` equal consecutive parts, each normalised by its own
// statistics; gain and bias span the whole row.  A block then takes one part of one row.
// One block a row; the order of a row's additions depends on the row's width only, so a row's
// bits do not depend on what else is in the step.
#include "common.cuh"

SGLC_DEFINE_ERROR_STRING()

enum { NORM_LAYER = 0, NORM_RMS = 1, NORM_COPY = 2 };   // NORM_COPY: the tail's second stage only, no norm

// Four floats at a time (VEC: a 32-bit source whose rows, gains and destination can be read and
// written 16 bytes at a time).  A thread's order of additions differs between the two forms; which
// form runs depends on the row width and the alignment of the buffers, never on the step.
__device__ __forceinline__ float sum4(const float4& v) { return (v.x + v.y) + (v.z + v.w); }
__device__ __forceinline__ float sq4(const float4& v, float mean, float q) {
  float d = v.x - mean; q = fmaf(d, d, q);
  d = v.y - mean; q = fmaf(d, d, q);
  d = v.z - mean; q = fmaf(d, d, q);
  d = v.w - mean; q = fmaf(d, d, q);
  return q;
}
__device__ __forceinline__ float4 norm4(const float4& v, float mean, float inv, const float* gain, const float* bias, int i) {
  float4 y = make_float4(__fmul_rn(v.x - mean, inv), __fmul_rn(v.y - mean, inv), __fmul_rn(v.z - mean, inv),
                         __fmul_rn(v.w - mean, inv));
  if (gain) {
    const float4 g = reinterpret_cast<const float4*>(gain)[i];
    y = make_float4(__fmul_rn(y.x, g.x), __fmul_rn(y.y, g.y), __fmul_rn(y.z, g.z), __fmul_rn(y.w, g.w));
  }
  if (bias) {
    const float4 b = reinterpret_cast<const float4*>(bias)[i];
    y = make_float4(__fadd_rn(y.x, b.x), __fadd_rn(y.y, b.y), __fadd_rn(y.z, b.z), __fadd_rn(y.w, b.w));
  }
  return y;
}
template <typename TO>
__device__ __forceinline__ void store4(TO* p, const float4& y) {
  if constexpr (sizeof(TO) == 4) {
    *reinterpret_cast<float4*>(p) = y;
  } else {
    __nv_bfloat162 h0 = __floats2bfloat162_rn(y.x, y.y), h1 = __floats2bfloat162_rn(y.z, y.w);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<uint32_t*>(&h0), *reinterpret_cast<uint32_t*>(&h1));
  }
}

template <typename TI, typename TO, bool ADD, bool VEC>
__global__ void norm_rows_kernel(const TI* __restrict__ src, long long src_stride,
                                 const int* __restrict__ src_rows, const float* __restrict__ gain, const float* __restrict__ bias,
                                 TO* __restrict__ dst, long long dst_stride, const int* __restrict__ dst_rows,
                                 int n_rows, int E, float eps, int form, long long dst_row_limit,
                                 int* __restrict__ err, int groups) {
  extern __shared__ __align__(16) float srow[];   // E floats
  __shared__ float red[33];
  // (groups > 1: a block takes one of a row's equal consecutive parts, E being the part's width)
  const int r = blockIdx.x / groups, part = (blockIdx.x % groups) * E;
  if (r >= n_rows) return;
  if (gain) gain += part;
  if (bias) bias += part;
  pdl_launch_dependents();
  pdl_wait();
  const TI* xr = src + (size_t)(src_rows ? src_rows[r] : r) * src_stride + part;
  float s = 0.0f;
  if constexpr (VEC) {
    for (int i = threadIdx.x; i < E / 4; i += blockDim.x) {
      const float4 v = reinterpret_cast<const float4*>(xr)[i];
      reinterpret_cast<float4*>(srow)[i] = v;
      s += sum4(v);
    }
  } else {
    for (int i = threadIdx.x; i < E; i += blockDim.x) {
      const float v = to_f32(xr[i]);
      srow[i] = v;
      s += v;
    }
  }
  float mean = 0.0f;
  if (form == NORM_LAYER) mean = block_sum(s, red) / (float)E;
  else __syncthreads();
  float q = 0.0f;
  if constexpr (VEC) {
    for (int i = threadIdx.x; i < E / 4; i += blockDim.x) q = sq4(reinterpret_cast<const float4*>(srow)[i], mean, q);
  } else {
    for (int i = threadIdx.x; i < E; i += blockDim.x) {
      const float d = srow[i] - mean;
      q = fmaf(d, d, q);
    }
  }
  const float inv = 1.0f / sqrtf(block_sum(q, red) / (float)E + eps);
  long long row = r;
  if (dst_rows) {
    row = dst_rows[r];
    if (row < 0 || !sglc_index_ok(row, dst_row_limit, err)) return;
  }
  TO* o = dst + (size_t)row * dst_stride + part;
  if constexpr (VEC) {
    for (int i = threadIdx.x; i < E / 4; i += blockDim.x) {
      float4 y = norm4(reinterpret_cast<const float4*>(srow)[i], mean, inv, gain, bias, i);
      if constexpr (ADD) {
        const float4 x = reinterpret_cast<const float4*>(o)[i];
        y = make_float4(__fadd_rn(x.x, y.x), __fadd_rn(x.y, y.y), __fadd_rn(x.z, y.z), __fadd_rn(x.w, y.w));
      }
      store4<TO>(o + 4 * i, y);
    }
  } else {
    for (int i = threadIdx.x; i < E; i += blockDim.x) {
      // (explicit roundings: the fused tail below must give the same bits, whatever either compiles to)
      float y = __fmul_rn(srow[i] - mean, inv);
      if (gain) y = __fmul_rn(y, gain[i]);
      if (bias) y = __fadd_rn(y, bias[i]);
      if (ADD) o[i] = from_f32<TO>(__fadd_rn(to_f32(o[i]), y));
      else o[i] = from_f32<TO>(y);
    }
  }
}

// The tail of a sublayer in one launch, a block a row:
//   x += norm_post(y) * g_post                                   (x: the 32-bit stream)
//   [mix]   hist[n_terms-1] = x;  x = sum_j w[j] * hist[j]        (a depth-weighted average, j ascending)
//   [next]  h = norm_next(x) * g_next                            (the norm ahead of the next sublayer;
//                                                                  form NORM_COPY: h = x in h's precision)
// The same arithmetic in the same order as the three kernels it stands for, so the bits are theirs.
template <typename TO, bool VEC>
__global__ void norm_add_tail_kernel(const float* __restrict__ y, long long y_stride,
                                     const float* __restrict__ g_post, float eps_post, int form_post,
                                     float* __restrict__ x, float* __restrict__ hist, long long hist_block,
                                     int n_terms, const float* __restrict__ mix_w,
                                     const float* __restrict__ g_next, float eps_next, int form_next,
                                     TO* __restrict__ h, long long h_stride, int n_rows, int E) {
  extern __shared__ __align__(16) float srow[];   // E floats
  __shared__ float red[33];
  const int r = blockIdx.x;
  if (r >= n_rows) return;
  pdl_launch_dependents();
  pdl_wait();
  const float* yr = y + (size_t)r * y_stride;
  const int n_it = VEC ? E / 4 : E;
  float s = 0.0f;
  for (int i = threadIdx.x; i < n_it; i += blockDim.x) {
    if constexpr (VEC) {
      const float4 v = reinterpret_cast<const float4*>(yr)[i];
      reinterpret_cast<float4*>(srow)[i] = v;
      s += sum4(v);
    } else {
      const float v = yr[i];
      srow[i] = v;
      s += v;
    }
  }
  float mean = 0.0f;
  if (form_post == NORM_LAYER) mean = block_sum(s, red) / (float)E;
  else __syncthreads();
  float q = 0.0f;
  for (int i = threadIdx.x; i < n_it; i += blockDim.x) {
    if constexpr (VEC) {
      q = sq4(reinterpret_cast<const float4*>(srow)[i], mean, q);
    } else {
      const float d = srow[i] - mean;
      q = fmaf(d, d, q);
    }
  }
  float inv = 1.0f / sqrtf(block_sum(q, red) / (float)E + eps_post);
  float* xr = x + (size_t)r * E;
  s = 0.0f;
  for (int i = threadIdx.x; i < n_it; i += blockDim.x) {
    if constexpr (VEC) {
      float4 v = norm4(reinterpret_cast<const float4*>(srow)[i], mean, inv, g_post, nullptr, i);
      const float4 x0 = reinterpret_cast<const float4*>(xr)[i];
      v = make_float4(__fadd_rn(x0.x, v.x), __fadd_rn(x0.y, v.y), __fadd_rn(x0.z, v.z), __fadd_rn(x0.w, v.w));
      if (n_terms > 0) {
        const size_t at = ((size_t)r * E) / 4 + i;
        reinterpret_cast<float4*>(hist + (size_t)(n_terms - 1) * hist_block)[at] = v;
        if (n_terms > 1) {
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int j = 0; j < n_terms - 1; j++) {
            const float4 hv = reinterpret_cast<const float4*>(hist + (size_t)j * hist_block)[at];
            const float wj = mix_w[j];
            acc.x = fmaf(wj, hv.x, acc.x); acc.y = fmaf(wj, hv.y, acc.y);
            acc.z = fmaf(wj, hv.z, acc.z); acc.w = fmaf(wj, hv.w, acc.w);
          }
          const float wl = mix_w[n_terms - 1];
          v = make_float4(fmaf(wl, v.x, acc.x), fmaf(wl, v.y, acc.y), fmaf(wl, v.z, acc.z), fmaf(wl, v.w, acc.w));
        }
      }
      reinterpret_cast<float4*>(xr)[i] = v;
      reinterpret_cast<float4*>(srow)[i] = v;
      s += sum4(v);
    } else {
      float v = __fmul_rn(srow[i] - mean, inv);
      if (g_post) v = __fmul_rn(v, g_post[i]);
      v = __fadd_rn(xr[i], v);
      if (n_terms > 0) {
        const size_t at = (size_t)r * E + i;
        hist[(size_t)(n_terms - 1) * hist_block + at] = v;
        if (n_terms > 1) {
          float acc = 0.0f;
          for (int j = 0; j < n_terms - 1; j++) acc = fmaf(mix_w[j], hist[(size_t)j * hist_block + at], acc);
          v = fmaf(mix_w[n_terms - 1], v, acc);
        }
      }
      xr[i] = v;
      srow[i] = v;
      s += v;
    }
  }
  if (!h) return;
  if (form_next == NORM_COPY) {
    __syncthreads();
    TO* hc = h + (size_t)r * h_stride;
    for (int i = threadIdx.x; i < n_it; i += blockDim.x) {
      if constexpr (VEC) store4<TO>(hc + 4 * i, reinterpret_cast<const float4*>(srow)[i]);
      else hc[i] = from_f32<TO>(srow[i]);
    }
    return;
  }
  mean = 0.0f;
  if (form_next == NORM_LAYER) mean = block_sum(s, red) / (float)E;
  else __syncthreads();
  q = 0.0f;
  for (int i = threadIdx.x; i < n_it; i += blockDim.x) {
    if constexpr (VEC) {
      q = sq4(reinterpret_cast<const float4*>(srow)[i], mean, q);
    } else {
      const float d = srow[i] - mean;
      q = fmaf(d, d, q);
    }
  }
  inv = 1.0f / sqrtf(block_sum(q, red) / (float)E + eps_next);
  TO* hr = h + (size_t)r * h_stride;
  for (int i = threadIdx.x; i < n_it; i += blockDim.x) {
    if constexpr (VEC) {
      store4<TO>(hr + 4 * i, norm4(reinterpret_cast<const float4*>(srow)[i], mean, inv, g_next, nullptr, i));
    } else {
      float v = __fmul_rn(srow[i] - mean, inv);
      if (g_next) v = __fmul_rn(v, g_next[i]);
      hr[i] = from_f32<TO>(v);
    }
  }
}

// y: float [n_rows][y_stride]; x: float [n_rows][E] contiguous; hist (n_terms > 0): float blocks of
// hist_block elements, block j holding [n_rows][E]; h (may be null): [n_rows][h_stride] of h_dtype.
static inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

SGLC_API int sglc_norm_add_tail(const float* y, long long y_stride, const float* g_post, float eps_post,
                                int form_post, float* x, float* hist, long long hist_block, int n_terms,
                                const float* mix_w, const float* g_next, float eps_next, int form_next, void* h,
                                long long h_stride, int h_dtype, int n_rows, int E, cudaStream_t stream) {
  if (n_rows <= 0) return SGLC_OK;
  if (E <= 0 || n_terms < 0 || (n_terms > 0 && !hist) || (n_terms > 1 && !mix_w)) return SGLC_ERR_ARGUMENT;
  if (h && h_dtype != SGLC_F32 && h_dtype != SGLC_BF16) return SGLC_ERR_ARGUMENT;
  const size_t smem = (size_t)E * sizeof(float);
  if (smem > 200 * 1024) return SGLC_ERR_UNSUPPORTED;
  const int threads = E >= 2048 ? 512 : (E >= 512 ? 256 : (E >= 128 ? 128 : (E >= 64 ? 64 : 32)));
  const bool vec = E % 4 == 0 && y_stride % 4 == 0 && al16(y) && al16(x) && al16(g_post) && al16(g_next) &&
                   (!hist || (al16(hist) && hist_block % 4 == 0)) &&
                   (!h || (h_stride % 4 == 0 && (reinterpret_cast<uintptr_t>(h) & (h_dtype == SGLC_F32 ? 15 : 7)) == 0));
#define TAIL(TO, VEC)                                                                                          \
  do {                                                                                                         \
    if (smem > 48 * 1024)                                                                                      \
      cudaFuncSetAttribute(norm_add_tail_kernel<TO, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    return sglc_launch(norm_add_tail_kernel<TO, VEC>, dim3(n_rows), dim3(threads), smem, stream, 1, true, y,    \
                       y_stride, g_post, eps_post, form_post, x, hist, hist_block, n_terms, mix_w, g_next,      \
                       eps_next, form_next, (TO*)h, h_stride, n_rows, E);                                       \
  } while (0)
  if (h && h_dtype == SGLC_BF16) {
    if (vec) TAIL(__nv_bfloat16, true);
    TAIL(__nv_bfloat16, false);
  }
  if (vec) TAIL(float, true);
  TAIL(float, false);
#undef TAIL
}

// form: 0 layer, 1 RMS.  src_rows: null, or the source row of every output row (a gather).  src_dtype/dst_dtype: SGLC_F32 or SGLC_BF16.  dst_rows: null, or the
// destination row of every source row (negative: the row is skipped); dst_row_limit: rows the
// destination holds (the bounds-check build compares).  add != 0: dst (float) += y.
SGLC_API int sglc_norm_rows_grouped(const void* src, long long src_stride, int src_dtype, const int* src_rows,
                                    const float* gain,
                                    const float* bias, void* dst, long long dst_stride, int dst_dtype,
                                    const int* dst_rows, long long dst_row_limit, int n_rows, int E_row, float eps,
                                    int form, int add, int groups, int* err, cudaStream_t stream) {
  if (n_rows <= 0) return SGLC_OK;
  if (E_row <= 0 || groups <= 0 || E_row % groups != 0 || (form != NORM_LAYER && form != NORM_RMS)) return SGLC_ERR_ARGUMENT;
  if ((long long)n_rows * groups > 0x7fffffffLL) return SGLC_ERR_UNSUPPORTED;
  const int E = E_row / groups;            // what a block normalises
  if (add && dst_dtype != SGLC_F32) return SGLC_ERR_ARGUMENT;
  const size_t smem = (size_t)E * sizeof(float);
  if (smem > 200 * 1024) return SGLC_ERR_UNSUPPORTED;
  const bool vec = src_dtype == SGLC_F32 && E % 4 == 0 && src_stride % 4 == 0 && dst_stride % 4 == 0 && al16(src) &&
                   al16(gain) && al16(bias) &&
                   (reinterpret_cast<uintptr_t>(dst) & (dst_dtype == SGLC_F32 ? 15 : 7)) == 0;
  // (a narrow part read four floats a thread fills no second warp: one warp then, whose sums are the
  // same bits, since the second warp only added zeros)
  const int threads = E >= 2048 ? 512 : (E >= 512 ? 256 : (E >= 128 ? 128 : (E >= 64 && !vec ? 64 : 32)));
#define LAUNCH(TI, TO, ADD) \
  do {                      \
    if (vec) LAUNCH_V(float, TO, ADD, true); \
    LAUNCH_V(TI, TO, ADD, false);            \
  } while (0)
#define LAUNCH_V(TI, TO, ADD, VEC)                                                                   \
  do {                                                                                               \
    if (smem > 48 * 1024)                                                                            \
      cudaFuncSetAttribute(norm_rows_kernel<TI, TO, ADD, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                           (int)smem);                                                               \
    return sglc_launch(norm_rows_kernel<TI, TO, ADD, VEC>, dim3(n_rows * groups), dim3(threads), smem, stream, 1, \
                       true, (const TI*)src, src_stride, src_rows, gain, bias, (TO*)dst, dst_stride, dst_rows,  \
                       n_rows, E, eps, form, dst_row_limit, err, groups);                             \
  } while (0)
  if (src_dtype == SGLC_F32) {
    if (add) LAUNCH(float, float, true);
    if (dst_dtype == SGLC_F32) LAUNCH(float, float, false);
    if (dst_dtype == SGLC_BF16) LAUNCH(float, __nv_bfloat16, false);
  } else if (src_dtype == SGLC_BF16) {
    if (add) LAUNCH(__nv_bfloat16, float, true);
    if (dst_dtype == SGLC_F32) LAUNCH(__nv_bfloat16, float, false);
    if (dst_dtype == SGLC_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16, false);
  }
#undef LAUNCH
#undef LAUNCH_V
  return SGLC_ERR_ARGUMENT;
}

SGLC_API int sglc_norm_rows(const void* src, long long src_stride, int src_dtype, const int* src_rows,
                            const float* gain,
                            const float* bias, void* dst, long long dst_stride, int dst_dtype,
                            const int* dst_rows, long long dst_row_limit, int n_rows, int E, float eps,
                            int form, int add, int* err, cudaStream_t stream) {
  return sglc_norm_rows_grouped(src, src_stride, src_dtype, src_rows, gain, bias, dst, dst_stride, dst_dtype, dst_rows,
                                dst_row_limit, n_rows, E, eps, form, add, 1, err, stream);
}
