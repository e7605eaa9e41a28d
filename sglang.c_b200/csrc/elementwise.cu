// Element-wise operations on the rows of a step.
//
// Depth mix: a model that hands every layer a weighted sum of all earlier layers' results keeps
// those results for the step's tokens, hist[j] (j = 0: the embedding output; j = i + 1: the
// result of layer i), as consecutive [n] blocks of 32-bit floats.  After layer i:
//   hist[i+1] = x;   x = sum_{j=0..i+1} w[j] * hist[j]      (32-bit, j ascending)
// with n_terms = i + 2.  n_terms = 1 only saves x as hist[0].
//
// Activation: y = act(x) for the activations that carry parameters of their own, where the
// product ahead has no epilogue for them.  xIELU with the two numbers ap > 0, an:
//   x > 0:   ap x^2 + x/2
//   x <= 0:  an (exp(x) - 1 - x) + x/2
#include "common.cuh"

SGLC_DEFINE_ERROR_STRING()

// VEC: n is a multiple of 4, so every hist block is 16-byte aligned and four elements go a load
template <bool VEC>
__global__ void depth_mix_kernel(float* __restrict__ x, float* __restrict__ hist, long long n,
                                 int n_terms, const float* __restrict__ w) {
  pdl_launch_dependents();
  pdl_wait();
  const long long n4 = VEC ? n / 4 : 0;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
       i += (long long)gridDim.x * blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(x)[i];
    reinterpret_cast<float4*>(hist + (size_t)(n_terms - 1) * n)[i] = v;
    if (n_terms > 1) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int j = 0; j < n_terms - 1; j++) {
        const float4 h = reinterpret_cast<const float4*>(hist + (size_t)j * n)[i];
        const float wj = w[j];
        acc.x = fmaf(wj, h.x, acc.x); acc.y = fmaf(wj, h.y, acc.y);
        acc.z = fmaf(wj, h.z, acc.z); acc.w = fmaf(wj, h.w, acc.w);
      }
      const float wl = w[n_terms - 1];
      acc.x = fmaf(wl, v.x, acc.x); acc.y = fmaf(wl, v.y, acc.y);
      acc.z = fmaf(wl, v.z, acc.z); acc.w = fmaf(wl, v.w, acc.w);
      reinterpret_cast<float4*>(x)[i] = acc;
    }
  }
  for (long long i = n4 * 4 + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float v = x[i];
    hist[(size_t)(n_terms - 1) * n + i] = v;
    if (n_terms > 1) {
      float acc = 0.0f;
      for (int j = 0; j < n_terms - 1; j++) acc = fmaf(w[j], hist[(size_t)j * n + i], acc);
      x[i] = fmaf(w[n_terms - 1], v, acc);
    }
  }
}

// x: [n] floats (the step's residual rows); hist: [n_terms and more][n]; w: [n_terms] floats
SGLC_API int sglc_depth_mix(float* x, float* hist, long long n, int n_terms, const float* w,
                            cudaStream_t stream) {
  if (n <= 0) return SGLC_OK;
  if (n_terms < 1 || (n_terms > 1 && !w)) return SGLC_ERR_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(hist) & 15)) return SGLC_ERR_ARGUMENT;
  const bool vec = n % 4 == 0;
  const long long work = vec ? n / 4 : n;
  int blocks = (int)((work + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (vec) return sglc_launch(depth_mix_kernel<true>, dim3(blocks), dim3(256), 0, stream, 1, true, x, hist, n, n_terms, w);
  return sglc_launch(depth_mix_kernel<false>, dim3(blocks), dim3(256), 0, stream, 1, true, x, hist, n, n_terms, w);
}

template <typename TI, typename TO>
__global__ void xielu_kernel(const TI* __restrict__ src, long long src_stride, TO* __restrict__ dst,
                             long long dst_stride, int rows, int cols, float ap, float an) {
  pdl_launch_dependents();
  pdl_wait();
  const long long total = (long long)rows * cols;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / cols, c = i % cols;
    dst[r * dst_stride + c] = from_f32<TO>(xielu_f32(to_f32(src[r * src_stride + c]), ap, an));
  }
}

SGLC_API int sglc_xielu(const void* src, long long src_stride, int src_dtype, void* dst,
                        long long dst_stride, int dst_dtype, int rows, int cols, float ap, float an,
                        cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return SGLC_OK;
  const long long total = (long long)rows * cols;
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
#define LAUNCH(TI, TO)                                                                              \
  return sglc_launch(xielu_kernel<TI, TO>, dim3(blocks), dim3(256), 0, stream, 1, true, (const TI*)src, \
                     src_stride, (TO*)dst, dst_stride, rows, cols, ap, an)
  if (src_dtype == SGLC_F32 && dst_dtype == SGLC_F32) LAUNCH(float, float);
  if (src_dtype == SGLC_F32 && dst_dtype == SGLC_BF16) LAUNCH(float, __nv_bfloat16);
  if (src_dtype == SGLC_BF16 && dst_dtype == SGLC_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
#undef LAUNCH
  return SGLC_ERR_ARGUMENT;
}

// Gated activation of a feed-forward whose gate and up projections are one product:
//   dst[r][j] = silu(src[r][j]) * src[r][F + j] * (w ? w[r][j / per] : 1),   j < F
// src holds the F gate columns, then the F up columns.  With `w` (float [rows][F / per]) a block of
// `per` columns is one expert of a mixture and takes the token's weight for it (zero: not chosen);
// columns from `n_weighted` on (an expert that every token uses, laid behind the routed ones) take 1.
// `act` chooses the gate's function (silu, or the tanh form of GELU); `mult` is one more factor of
// every result (a layer's residual multiplier, taken in 32-bit ahead of the rounding).
enum { GA_SILU = 0, GA_GELU_TANH = 1 };
template <typename TI, typename TO>
__global__ void gated_act_kernel(const TI* __restrict__ src, long long src_stride, TO* __restrict__ dst,
                                 long long dst_stride, int rows, int F, const float* __restrict__ w,
                                 long long w_stride, int per, int act, float mult, int n_weighted) {
  pdl_launch_dependents();
  pdl_wait();
  const long long total = (long long)rows * F;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / F;
    const int c = (int)(i % F);
    const float wt = (w && c < n_weighted) ? w[r * w_stride + c / per] : 1.0f;
    float out = 0.0f;
    if (wt != 0.0f) {
      const float g = to_f32(src[r * src_stride + c]), u = to_f32(src[r * src_stride + F + c]);
      out = (act == GA_GELU_TANH ? gelu_tanh_f32(g) : g / (1.0f + expf(-g))) * u * (wt * mult);
    }
    dst[r * dst_stride + c] = from_f32<TO>(out);
  }
}

// bfloat16 in and out, eight columns a thread (16-byte loads and stores): F, the strides and `per`
// multiples of 8, rows 16-byte aligned
__global__ void gated_act_vec8_kernel(const __nv_bfloat16* __restrict__ src, long long src_stride,
                                      __nv_bfloat16* __restrict__ dst, long long dst_stride, int rows, int F,
                                      const float* __restrict__ w, long long w_stride, int per, int act, float mult,
                                      int n_weighted) {
  pdl_launch_dependents();
  pdl_wait();
  const int F8 = F / 8;
  const long long total = (long long)rows * F8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / F8;
    const int c = (int)(i % F8) * 8;
    const float wt = ((w && c < n_weighted) ? w[r * w_stride + c / per] : 1.0f) * mult;
    uint4 o = make_uint4(0u, 0u, 0u, 0u);
    if (wt != 0.0f) {
      const uint4 g4 = *reinterpret_cast<const uint4*>(src + r * src_stride + c);
      const uint4 u4 = *reinterpret_cast<const uint4*>(src + r * src_stride + F + c);
      const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g4);
      const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&u4);
      __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int k = 0; k < 4; k++) {
        const float2 g = __bfloat1622float2(gp[k]), u = __bfloat1622float2(up[k]);
        if (act == GA_GELU_TANH)
          op[k] = __floats2bfloat162_rn(gelu_tanh_f32(g.x) * u.x * wt, gelu_tanh_f32(g.y) * u.y * wt);
        else
          op[k] = __floats2bfloat162_rn(g.x / (1.0f + expf(-g.x)) * u.x * wt, g.y / (1.0f + expf(-g.y)) * u.y * wt);
      }
    }
    *reinterpret_cast<uint4*>(dst + r * dst_stride + c) = o;
  }
}

// n_weighted: the first so many columns (a multiple of `per`) take weights, the rest take 1
SGLC_API int sglc_gated_act_part(const void* src, long long src_stride, int src_dtype, void* dst, long long dst_stride,
                                 int dst_dtype, int rows, int F, const float* w, long long w_stride, int per,
                                 int act, float mult, int n_weighted, cudaStream_t stream) {
  if (rows <= 0 || F <= 0) return SGLC_OK;
  if (act != GA_SILU && act != GA_GELU_TANH) return SGLC_ERR_ARGUMENT;
  if (w && (per <= 0 || n_weighted < 0 || n_weighted > F || n_weighted % per != 0)) return SGLC_ERR_ARGUMENT;
  const long long total = (long long)rows * F;
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (src_dtype == SGLC_BF16 && dst_dtype == SGLC_BF16 && F % 8 == 0 && src_stride % 8 == 0 && dst_stride % 8 == 0 &&
      (!w || (per % 8 == 0 && n_weighted % 8 == 0)) && (((uintptr_t)src | (uintptr_t)dst) & 15) == 0) {
    int b8 = (int)((total / 8 + 255) / 256);
    if (b8 > 148 * 16) b8 = 148 * 16;
    return sglc_launch(gated_act_vec8_kernel, dim3(b8), dim3(256), 0, stream, 1, true, (const __nv_bfloat16*)src,
                       src_stride, (__nv_bfloat16*)dst, dst_stride, rows, F, w, w_stride, per > 0 ? per : 1, act, mult,
                       n_weighted);
  }
#define LAUNCH(TI, TO)                                                                                  \
  return sglc_launch(gated_act_kernel<TI, TO>, dim3(blocks), dim3(256), 0, stream, 1, true, (const TI*)src, \
                     src_stride, (TO*)dst, dst_stride, rows, F, w, w_stride, per > 0 ? per : 1, act, mult, n_weighted)
  if (src_dtype == SGLC_F32 && dst_dtype == SGLC_F32) LAUNCH(float, float);
  if (src_dtype == SGLC_F32 && dst_dtype == SGLC_BF16) LAUNCH(float, __nv_bfloat16);
  if (src_dtype == SGLC_BF16 && dst_dtype == SGLC_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
#undef LAUNCH
  return SGLC_ERR_ARGUMENT;
}

SGLC_API int sglc_gated_act_ext(const void* src, long long src_stride, int src_dtype, void* dst, long long dst_stride,
                                int dst_dtype, int rows, int F, const float* w, long long w_stride, int per,
                                int act, float mult, cudaStream_t stream) {
  if (w && (per <= 0 || F % per != 0)) return SGLC_ERR_ARGUMENT;
  return sglc_gated_act_part(src, src_stride, src_dtype, dst, dst_stride, dst_dtype, rows, F, w, w_stride, per, act,
                             mult, F, stream);
}

SGLC_API int sglc_gated_act(const void* src, long long src_stride, int src_dtype, void* dst, long long dst_stride,
                            int dst_dtype, int rows, int F, const float* w, long long w_stride, int per,
                            cudaStream_t stream) {
  return sglc_gated_act_ext(src, src_stride, src_dtype, dst, dst_stride, dst_dtype, rows, F, w, w_stride, per, GA_SILU,
                            1.0f, stream);
}

// 32-bit rows into a column range of rows of another precision: dst[r][j] = src[r][j], j < cols
// (the operand of a product made of several streams laid side by side).
template <typename TO>
__global__ void cast_rows_kernel(const float* __restrict__ src, long long src_stride, TO* __restrict__ dst,
                                 long long dst_stride, int rows, int cols) {
  pdl_launch_dependents();
  pdl_wait();
  const long long total = (long long)rows * cols;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / cols, c = i % cols;
    dst[r * dst_stride + c] = from_f32<TO>(src[r * src_stride + c]);
  }
}

SGLC_API int sglc_cast_rows(const float* src, long long src_stride, void* dst, long long dst_stride, int dst_dtype,
                            int rows, int cols, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return SGLC_OK;
  const long long total = (long long)rows * cols;
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dst_dtype == SGLC_F32)
    return sglc_launch(cast_rows_kernel<float>, dim3(blocks), dim3(256), 0, stream, 1, true, src, src_stride,
                       (float*)dst, dst_stride, rows, cols);
  if (dst_dtype == SGLC_BF16)
    return sglc_launch(cast_rows_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, 1, true, src, src_stride,
                       (__nv_bfloat16*)dst, dst_stride, rows, cols);
  return SGLC_ERR_ARGUMENT;
}

// A gate times a row of a token table: dst[t][j] = act(z[t][j]) * table[tokens[t]][first + j], j < cols
// (act: the tanh form of GELU).  z: 32-bit rows; the table float or bfloat16 with rows of `table_cols`;
// a token id outside the table raises the error word and gives zeros.
template <typename TW, typename TO>
__global__ void gated_gather_kernel(const float* __restrict__ z, long long z_stride, const int* __restrict__ tokens,
                                    const TW* __restrict__ table, long long table_cols, int n_table_rows, int first,
                                    TO* __restrict__ dst, long long dst_stride, int rows, int cols,
                                    int* __restrict__ err) {
  pdl_launch_dependents();
  pdl_wait();
  const long long total = (long long)rows * cols;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / cols;
    const int c = (int)(i % cols);
    const int tok = tokens[r];
    float out = 0.0f;
    if (tok >= 0 && tok < n_table_rows)
      out = gelu_tanh_f32(z[r * z_stride + c]) * to_f32(table[(size_t)tok * table_cols + first + c]);
    else if (err)
      atomicExch(err, 1);
    dst[r * dst_stride + c] = from_f32<TO>(out);
  }
}

SGLC_API int sglc_gated_gather(const float* z, long long z_stride, const int* tokens, const void* table,
                               long long table_cols, int n_table_rows, int first, int table_dtype, void* dst,
                               long long dst_stride, int dst_dtype, int rows, int cols, int* err, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return SGLC_OK;
  if (first < 0 || first + cols > table_cols || n_table_rows <= 0) return SGLC_ERR_ARGUMENT;
  const long long total = (long long)rows * cols;
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
#define LAUNCH(TW, TO)                                                                                        \
  return sglc_launch(gated_gather_kernel<TW, TO>, dim3(blocks), dim3(256), 0, stream, 1, true, z, z_stride, tokens, \
                     (const TW*)table, table_cols, n_table_rows, first, (TO*)dst, dst_stride, rows, cols, err)
  if (table_dtype == SGLC_F32 && dst_dtype == SGLC_F32) LAUNCH(float, float);
  if (table_dtype == SGLC_BF16 && dst_dtype == SGLC_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  if (table_dtype == SGLC_BF16 && dst_dtype == SGLC_F32) LAUNCH(__nv_bfloat16, float);
  if (table_dtype == SGLC_F32 && dst_dtype == SGLC_BF16) LAUNCH(float, __nv_bfloat16);
#undef LAUNCH
  return SGLC_ERR_ARGUMENT;
}
