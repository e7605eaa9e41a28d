// Rotary positions for the queries and keys of a step, the unit-RMS norm behind them, and the
// write of the new keys and values into their cache pages, in one launch.
//
// A head's first `dims` entries are turned in pairs (i, i + dims/2), the "rotate half" layout:
//   (u, v) -> (u cos a - v sin a,  v cos a + u sin a),   a = position * f_i,
// cos and sin both times `mult`; the remaining entries pass.  The frequencies f_i (dims/2 of
// them, made once by the host in 64-bit, whatever scaling rule shaped them) arrive as a table;
// the angle is formed in 64-bit and brought into one turn before the 32-bit sine and cosine.
// With `norm` the turned head is divided by its root mean square (eps inside the root, no gain).
//
// Input: 32-bit rows x [T][..] holding H query heads of D, then G key heads of D, then G value
// heads of V.  Queries leave as [T][H*D] in the activation precision; keys and values go to
// cache[page][ G x page_size x D keys | G x page_size x V values ] at slots[t] = page *
// page_size + offset (a page with equal D and V is the usual [2][G][page_size][D]).
#include "common.cuh"

SGLC_DEFINE_ERROR_STRING()

constexpr int ROT_WARPS = 4;
constexpr int ROT_MAX_DIM = 512;

template <typename TA>
__global__ void __launch_bounds__(ROT_WARPS * 32)
rotary_kv_kernel(const float* __restrict__ x, long long x_stride, const int* __restrict__ positions,
                 const double* __restrict__ freq, float mult, int dims, int norm, float eps,
                 TA* __restrict__ q_out, long long q_stride, TA* __restrict__ cache, const int* __restrict__ slots,
                 int T, int H, int G, int D, int V, int page_size, int n_pages, int* err) {
  __shared__ float buf[ROT_WARPS][ROT_MAX_DIM];
  pdl_launch_dependents();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_wait();
  const int pos = positions[t];
  const int slot = slots[t];
  const int page = slot / page_size, off = slot % page_size;
  const bool page_ok = slot >= 0 && sglc_index_ok(page, n_pages, err);
  const size_t page_elems = (size_t)G * page_size * (D + V);
  const float* xr = x + (size_t)t * x_stride;
  const int half = dims / 2;
  float* b = buf[warp];
  for (int row = warp; row < H + 2 * G; row += ROT_WARPS) {
    if (row >= H + G) {                        // a value head: copied
      const int g = row - H - G;
      if (page_ok) {
        TA* dst = cache + (size_t)page * page_elems + (size_t)G * page_size * D + ((size_t)g * page_size + off) * V;
        const float* src = xr + (size_t)(H + G) * D + (size_t)g * V;
        for (int d = lane; d < V; d += 32) dst[d] = from_f32<TA>(src[d]);
      }
      continue;
    }
    const float* src = xr + (size_t)row * D;
    float ss = 0.0f;
    for (int i = lane; i < half; i += 32) {
      double a = (double)pos * freq[i];
      a -= floor(a * 0.15915494309189535) * 6.283185307179586;
      float sn, cs;
      sincosf((float)a, &sn, &cs);
      sn *= mult; cs *= mult;
      const float u = src[i], v = src[i + half];
      const float ru = u * cs - v * sn, rv = v * cs + u * sn;
      b[i] = ru; b[i + half] = rv;
      ss = fmaf(ru, ru, fmaf(rv, rv, ss));
    }
    for (int d = 2 * half + lane; d < D; d += 32) {
      const float u = src[d];
      b[d] = u;
      ss = fmaf(u, u, ss);
    }
    ss = warp_sum(ss);
    const float f = norm ? 1.0f / sqrtf(ss / (float)D + eps) : 1.0f;
    __syncwarp();
    TA* dst = nullptr;
    if (row < H) dst = q_out + (size_t)t * q_stride + (size_t)row * D;
    else if (page_ok) dst = cache + (size_t)page * page_elems + ((size_t)(row - H) * page_size + off) * D;
    if (dst)
      for (int d = lane; d < D; d += 32) dst[d] = from_f32<TA>(b[d] * f);
    __syncwarp();
  }
}

SGLC_API int sglc_rotary_kv(const float* x, long long x_stride, const int* positions, const double* freq, float mult,
                            int dims, int norm, float eps, void* q_out, long long q_stride, void* cache,
                            const int* slots, int T, int H, int G, int D, int V, int page_size, int n_pages,
                            int dtype, int* err, cudaStream_t stream) {
  if (T <= 0) return SGLC_OK;
  if (H <= 0 || G <= 0 || D <= 0 || V <= 0 || dims < 0 || dims > D || dims % 2 != 0 || page_size <= 0)
    return SGLC_ERR_ARGUMENT;
  if (D > ROT_MAX_DIM) return SGLC_ERR_UNSUPPORTED;
  if (dtype == SGLC_F32)
    return sglc_launch(rotary_kv_kernel<float>, dim3(T), dim3(ROT_WARPS * 32), 0, stream, 1, true, x, x_stride,
                       positions, freq, mult, dims, norm, eps, (float*)q_out, q_stride, (float*)cache, slots, T, H, G,
                       D, V, page_size, n_pages, err);
  if (dtype == SGLC_BF16)
    return sglc_launch(rotary_kv_kernel<__nv_bfloat16>, dim3(T), dim3(ROT_WARPS * 32), 0, stream, 1, true, x,
                       x_stride, positions, freq, mult, dims, norm, eps, (__nv_bfloat16*)q_out, q_stride,
                       (__nv_bfloat16*)cache, slots, T, H, G, D, V, page_size, n_pages, err);
  return SGLC_ERR_ARGUMENT;
}

// The input stage of a latent attention with a turned part, in one launch, a block a token:
//   every query head [R entries | Rd entries]: the first R pass (they are already in the latent's
//     coordinates), the last Rd are turned by the token's position;
//   the token's latent row `low` [R | Rd]: the first R are divided by their root mean square (eps
//     inside the root) and multiplied by a gain, the last Rd (one key part that all heads share)
//     are turned the same way; the row goes straight into the cache's rows at slots[t].
// Of the Rd entries the first `dims` are turned, the rest pass.  `pairing` 0: pairs (i, i + dims/2);
// 1: neighbours (2i, 2i + 1).  Angles as above: 64-bit, brought into one turn, then sincosf.
// Queries arrive as 32-bit rows and leave in the activation precision, which is the cache's.
template <typename TA>
__global__ void __launch_bounds__(ROT_WARPS * 32)
latent_rope_kernel(const float* __restrict__ qx, long long qx_stride, const float* __restrict__ low,
                   long long low_stride, const float* __restrict__ gain, float eps, const int* __restrict__ positions,
                   const double* __restrict__ freq, float mult, int dims, int pairing, TA* __restrict__ q_out,
                   long long q_stride, TA* __restrict__ rows, const int* __restrict__ slots, long long n_rows, int T,
                   int H, int R, int Rd, int* err) {
  pdl_launch_dependents();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_wait();
  const int pos = positions[t];
  const int half = dims / 2, W = R + Rd;
  for (int row = warp; row < H + (low ? 1 : 0); row += ROT_WARPS) {
    const float* src;
    TA* dst;
    if (row < H) {
      src = qx + (size_t)t * qx_stride + (size_t)row * W;
      dst = q_out + (size_t)t * q_stride + (size_t)row * W;
      for (int d = lane; d < R; d += 32) dst[d] = from_f32<TA>(src[d]);
    } else {
      const long long slot = slots[t];
      if (slot < 0 || !sglc_index_ok(slot, n_rows, err)) continue;
      src = low + (size_t)t * low_stride;
      dst = rows + (size_t)slot * W;
      float ss = 0.0f;
      for (int d = lane; d < R; d += 32) ss = fmaf(src[d], src[d], ss);
      ss = warp_sum(ss);
      const float inv = 1.0f / sqrtf(ss / (float)R + eps);
      for (int d = lane; d < R; d += 32) dst[d] = from_f32<TA>(src[d] * inv * gain[d]);
    }
    src += R;
    dst += R;
    for (int i = lane; i < half; i += 32) {
      double a = (double)pos * freq[i];
      a -= floor(a * 0.15915494309189535) * 6.283185307179586;
      float sn, cs;
      sincosf((float)a, &sn, &cs);
      sn *= mult; cs *= mult;
      const int iu = pairing ? 2 * i : i, iv = pairing ? 2 * i + 1 : i + half;
      const float u = src[iu], v = src[iv];
      dst[iu] = from_f32<TA>(u * cs - v * sn);
      dst[iv] = from_f32<TA>(v * cs + u * sn);
    }
    for (int d = 2 * half + lane; d < Rd; d += 32) dst[d] = from_f32<TA>(src[d]);
  }
}

// qx: float [T][H*(R+Rd)]; low: float [T][R+Rd] or null (a layer that reads latents another layer
// cached); gain: float [R]; q_out: [T][H*(R+Rd)]; rows: the cache seen as [n_rows][R+Rd].
SGLC_API int sglc_latent_rope(const float* qx, long long qx_stride, const float* low, long long low_stride,
                              const float* gain, float eps, const int* positions, const double* freq, float mult,
                              int dims, int pairing, void* q_out, long long q_stride, void* rows, const int* slots,
                              long long n_rows, int T, int H, int R, int Rd, int dtype, int* err,
                              cudaStream_t stream) {
  if (T <= 0) return SGLC_OK;
  if (H <= 0 || R <= 0 || Rd < 0 || dims < 0 || dims > Rd || dims % 2 != 0 || (low && (!gain || !rows || !slots)))
    return SGLC_ERR_ARGUMENT;
  if (dtype == SGLC_F32)
    return sglc_launch(latent_rope_kernel<float>, dim3(T), dim3(ROT_WARPS * 32), 0, stream, 1, true, qx, qx_stride, low,
                       low_stride, gain, eps, positions, freq, mult, dims, pairing, (float*)q_out, q_stride, (float*)rows,
                       slots, n_rows, T, H, R, Rd, err);
  if (dtype == SGLC_BF16)
    return sglc_launch(latent_rope_kernel<__nv_bfloat16>, dim3(T), dim3(ROT_WARPS * 32), 0, stream, 1, true, qx,
                       qx_stride, low, low_stride, gain, eps, positions, freq, mult, dims, pairing,
                       (__nv_bfloat16*)q_out, q_stride, (__nv_bfloat16*)rows, slots, n_rows, T, H, R, Rd, err);
  return SGLC_ERR_ARGUMENT;
}

// The general input stage of a softmax attention, a block a token: 32-bit rows x holding H query
// heads of D, then (with G > 0: a layer that owns its keys and values) G key heads of D and G value
// heads of V.  Per head, in this order:
//   norm (norm_mode)   0: none.  1: after the turn, the head divided by its root mean square, no gain.
//                      2: before the turn, the head divided by its root mean square times a gain of
//                         D entries that the heads share (gain_q for queries, gain_k for keys).
//                      3: before the turn, all query heads of the token divided by ONE root mean
//                         square over their H*D entries, times a gain of H*D entries (gain_q); the key
//                         heads likewise over G*D entries (gain_k).
//   turn               the first `dims` entries by position * freq[i], pairs (i, i + dims/2)
//                      (pairing 0) or (2i, 2i + 1) (pairing 1); the rest pass.
// Queries leave as [T][H*D] in the activation precision; keys and values go to their cache page
// (G x page_size x D keys, then G x page_size x V values) at slots[t]; values are multiplied by
// v_mult on the way (a mixer whose result is a fixed multiple of the attention's folds it here:
// the attention is linear in its values).  eps lies inside every root.
constexpr int QK_WARPS = 8;      // (a token's head rows are dealt to the warps: eight keep the rounds few)

template <typename TA>
__global__ void __launch_bounds__(QK_WARPS * 32)
qk_prep_kernel(const float* __restrict__ x, long long x_stride, const int* __restrict__ positions,
               const double* __restrict__ freq, float mult, int dims, int pairing, int norm_mode, float eps,
               const float* __restrict__ gain_q, const float* __restrict__ gain_k, float v_mult,
               TA* __restrict__ q_out, long long q_stride, TA* __restrict__ cache, const int* __restrict__ slots,
               int T, int H, int G, int D, int V, int page_size, int n_pages, int* err) {
  __shared__ float buf[QK_WARPS][ROT_MAX_DIM];
  __shared__ float red[2][QK_WARPS];
  pdl_launch_dependents();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_wait();
  const int pos = positions[t];
  const int slot = G > 0 ? slots[t] : -1;
  const int page = slot / page_size, off = slot % page_size;
  const bool page_ok = G > 0 && slot >= 0 && sglc_index_ok(page, n_pages, err);
  const size_t page_elems = (size_t)G * page_size * (D + V);
  const float* xr = x + (size_t)t * x_stride;
  const int half = dims / 2;
  float inv_all[2] = {1.0f, 1.0f};
  if (norm_mode == 3) {
    // one root mean square over all query heads, one over all key heads: every thread sums its
    // share in a fixed order, so a token's bits do not depend on the rest of the step
    float sq = 0.0f, sk = 0.0f;
    for (int i = threadIdx.x; i < H * D; i += QK_WARPS * 32) sq = fmaf(xr[i], xr[i], sq);
    for (int i = threadIdx.x; i < G * D; i += QK_WARPS * 32) sk = fmaf(xr[H * D + i], xr[H * D + i], sk);
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    if (lane == 0) { red[0][warp] = sq; red[1][warp] = sk; }
    __syncthreads();
    sq = 0.0f; sk = 0.0f;
    for (int w = 0; w < QK_WARPS; w++) { sq += red[0][w]; sk += red[1][w]; }
    inv_all[0] = 1.0f / sqrtf(sq / (float)(H * D) + eps);
    if (G > 0) inv_all[1] = 1.0f / sqrtf(sk / (float)(G * D) + eps);
  }
  float* b = buf[warp];
  for (int row = warp; row < H + 2 * G; row += QK_WARPS) {
    if (row >= H + G) {                        // a value head: copied (times v_mult)
      const int g = row - H - G;
      if (page_ok) {
        TA* dst = cache + (size_t)page * page_elems + (size_t)G * page_size * D + ((size_t)g * page_size + off) * V;
        const float* src = xr + (size_t)(H + G) * D + (size_t)g * V;
        for (int d = lane; d < V; d += 32) dst[d] = from_f32<TA>(src[d] * v_mult);
      }
      continue;
    }
    const bool is_q = row < H;
    const float* src = xr + (size_t)row * D;
    float ss = 0.0f;
    for (int d = lane; d < D; d += 32) {
      const float u = src[d];
      b[d] = u;
      ss = fmaf(u, u, ss);
    }
    if (norm_mode == 2) {
      ss = warp_sum(ss);
      const float inv = 1.0f / sqrtf(ss / (float)D + eps);
      const float* gn = is_q ? gain_q : gain_k;
      for (int d = lane; d < D; d += 32) b[d] = __fmul_rn(__fmul_rn(b[d], inv), gn[d]);
    } else if (norm_mode == 3) {
      const float inv = inv_all[is_q ? 0 : 1];
      const float* gn = is_q ? gain_q + (size_t)row * D : gain_k + (size_t)(row - H) * D;
      for (int d = lane; d < D; d += 32) b[d] = __fmul_rn(__fmul_rn(b[d], inv), gn[d]);
    }
    __syncwarp();
    ss = 0.0f;
    for (int i = lane; i < half; i += 32) {
      double a = (double)pos * freq[i];
      a -= floor(a * 0.15915494309189535) * 6.283185307179586;
      float sn, cs;
      sincosf((float)a, &sn, &cs);
      sn *= mult; cs *= mult;
      const int iu = pairing ? 2 * i : i, iv = pairing ? 2 * i + 1 : i + half;
      const float u = b[iu], v = b[iv];
      const float ru = u * cs - v * sn, rv = v * cs + u * sn;
      b[iu] = ru; b[iv] = rv;
      ss = fmaf(ru, ru, fmaf(rv, rv, ss));
    }
    float f = 1.0f;
    if (norm_mode == 1) {
      for (int d = 2 * half + lane; d < D; d += 32) ss = fmaf(b[d], b[d], ss);
      ss = warp_sum(ss);
      f = 1.0f / sqrtf(ss / (float)D + eps);
    }
    __syncwarp();
    TA* dst = nullptr;
    if (is_q) dst = q_out + (size_t)t * q_stride + (size_t)row * D;
    else if (page_ok) dst = cache + (size_t)page * page_elems + ((size_t)(row - H) * page_size + off) * D;
    if (dst)
      for (int d = lane; d < D; d += 32) dst[d] = from_f32<TA>(b[d] * f);
    __syncwarp();
  }
}

// x: float [T][H*D (+ G*D + G*V)]; G = 0: queries only (cache and slots unused); gain_q, gain_k:
// float, [D] each (norm_mode 2) or [H*D] and [G*D] (norm_mode 3), else unused.
SGLC_API int sglc_qk_prep(const float* x, long long x_stride, const int* positions, const double* freq, float mult,
                          int dims, int pairing, int norm_mode, float eps, const float* gain_q, const float* gain_k,
                          float v_mult, void* q_out, long long q_stride, void* cache, const int* slots, int T, int H,
                          int G, int D, int V, int page_size, int n_pages, int dtype, int* err, cudaStream_t stream) {
  if (T <= 0) return SGLC_OK;
  if (H <= 0 || G < 0 || D <= 0 || V <= 0 || dims < 0 || dims > D || dims % 2 != 0 || page_size <= 0 ||
      norm_mode < 0 || norm_mode > 3 || (pairing != 0 && pairing != 1))
    return SGLC_ERR_ARGUMENT;
  if (norm_mode >= 2 && (!gain_q || (G > 0 && !gain_k))) return SGLC_ERR_ARGUMENT;
  if (G > 0 && (!cache || !slots)) return SGLC_ERR_ARGUMENT;
  if (dims > 0 && !freq) return SGLC_ERR_ARGUMENT;
  if (D > ROT_MAX_DIM) return SGLC_ERR_UNSUPPORTED;
  if (dtype == SGLC_F32)
    return sglc_launch(qk_prep_kernel<float>, dim3(T), dim3(QK_WARPS * 32), 0, stream, 1, true, x, x_stride, positions,
                       freq, mult, dims, pairing, norm_mode, eps, gain_q, gain_k, v_mult, (float*)q_out, q_stride,
                       (float*)cache, slots, T, H, G, D, V, page_size, n_pages, err);
  if (dtype == SGLC_BF16)
    return sglc_launch(qk_prep_kernel<__nv_bfloat16>, dim3(T), dim3(QK_WARPS * 32), 0, stream, 1, true, x, x_stride,
                       positions, freq, mult, dims, pairing, norm_mode, eps, gain_q, gain_k, v_mult,
                       (__nv_bfloat16*)q_out, q_stride, (__nv_bfloat16*)cache, slots, T, H, G, D, V, page_size, n_pages,
                       err);
  return SGLC_ERR_ARGUMENT;
}
