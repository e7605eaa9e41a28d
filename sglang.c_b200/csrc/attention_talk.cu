// Softmax attention whose heads talk to one another after the softmax, over a paged cache that
// keeps ONE row per position and key/value head: the projected key before its norm, which is also
// the value.
//
//   q^_h = rms_norm(q_h) * wq,  k^_c = rms_norm(k_c) * wk            (per head, gains shared by the heads)
//   s_h(i, j) = (q^_h(i) . k^_c(j)) * scale - slope_h * (i - j)       c = h / (H / G);  0 <= i - j < window
//   p_h(i, .) = softmax over the visible j
//   p'_h(i, j) = sum_g talk[h][g] p_g(i, j)                           (the heads' weights mixed)
//   o_h(i) = sum_j p'_h(i, j) k_c(j)                                  (values: the keys as projected)
//   out = o * sigmoid(gate) * mult                                    (gate: one more projection of the layer's input)
//
// Two launches.  `talk_prep` (a block a token, a warp a head row): queries are divided by their
// root mean square and multiplied by wq * wk (the key's gain rides on the query: the cache holds
// plain keys), 32-bit; the keys go into their cache rows as they are.  `talk_attention` (a block a
// token, a warp a head): the key's own 1/rms is formed from the cached row beside the dot product.
// Mixing needs p, not exp(s - running max): so the keys are visited twice, first for every head's
// maximum and sum, then for the weights, which the warps exchange through shared memory tile by
// tile, mix, and apply to the values.  Tiles are 32 keys by absolute position (a lane a key), so a
// token's order of additions depends on its own position and window only: the same bits however the
// tokens were cut into steps and whatever else is in the step.  Scores, weights, sums: 32-bit.
#include "common.cuh"

SGLC_DEFINE_ERROR_STRING()

constexpr int TALK_MAX_HEADS = 32;
constexpr int TALK_MAX_DIM = 256;
constexpr int TALK_PREP_WARPS = 4;

template <typename TC>
__global__ void __launch_bounds__(TALK_PREP_WARPS * 32)
talk_prep_kernel(const float* __restrict__ x, long long x_stride, const float* __restrict__ wq,
                 const float* __restrict__ wk, float eps, float* __restrict__ q_out, long long q_stride,
                 TC* __restrict__ cache, const int* __restrict__ slots, int T, int H, int G, int D, int page_size,
                 int n_pages, int* err) {
  pdl_launch_dependents();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_wait();
  const int slot = slots[t];
  const int page = slot / page_size, off = slot % page_size;
  const bool page_ok = slot >= 0 && sglc_index_ok(page, n_pages, err);
  const float* xr = x + (size_t)t * x_stride;
  for (int row = warp; row < H + G; row += TALK_PREP_WARPS) {
    const float* src = xr + (size_t)row * D;
    if (row < H) {
      float ss = 0.0f;
      for (int d = lane; d < D; d += 32) ss = fmaf(src[d], src[d], ss);
      ss = warp_sum(ss);
      const float inv = 1.0f / sqrtf(ss / (float)D + eps);
      float* dst = q_out + (size_t)t * q_stride + (size_t)row * D;
      for (int d = lane; d < D; d += 32) dst[d] = src[d] * inv * (wq[d] * wk[d]);
    } else if (page_ok) {
      TC* dst = cache + ((size_t)page * G + (row - H)) * page_size * D + (size_t)off * D;
      for (int d = lane; d < D; d += 32) dst[d] = from_f32<TC>(src[d]);
    }
  }
}

__device__ __forceinline__ void talk_load4(const float* p, float* v) {
  const float4 x = *reinterpret_cast<const float4*>(p);
  v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
}
__device__ __forceinline__ void talk_load4(const __nv_bfloat16* p, float* v) {
  const uint2 x = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&x.x);
  const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&x.y);
  v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
}

// one key's score for one head: (q . k) / rms(k) * scale - slope * distance; kp: the key's row
template <typename TC>
__device__ __forceinline__ float talk_score(const float* __restrict__ qv, const TC* __restrict__ kp, int D, float eps,
                                            float scale, float bias) {
  float dot = 0.0f, kk = 0.0f;
  if (D % 4 == 0) {
    for (int d = 0; d < D; d += 4) {
      float k4[4];
      talk_load4(kp + d, k4);
      const float4 q4 = *reinterpret_cast<const float4*>(qv + d);
      dot = fmaf(q4.x, k4[0], dot); kk = fmaf(k4[0], k4[0], kk);
      dot = fmaf(q4.y, k4[1], dot); kk = fmaf(k4[1], k4[1], kk);
      dot = fmaf(q4.z, k4[2], dot); kk = fmaf(k4[2], k4[2], kk);
      dot = fmaf(q4.w, k4[3], dot); kk = fmaf(k4[3], k4[3], kk);
    }
  } else {
    for (int d = 0; d < D; d++) {
      const float kv = to_f32(kp[d]);
      dot = fmaf(qv[d], kv, dot);
      kk = fmaf(kv, kv, kk);
    }
  }
  return dot * (1.0f / sqrtf(kk / (float)D + eps)) * scale - bias;
}

// NV: output columns a lane keeps (D <= 32 NV)
template <typename TC, typename TO, int NV>
__global__ void __launch_bounds__(TALK_MAX_HEADS * 32)
talk_attention_kernel(const float* __restrict__ q, long long q_stride, const TC* __restrict__ cache,
                      const int* __restrict__ block_table, int bt_stride, const int* __restrict__ token_req,
                      const int* __restrict__ positions, const float* __restrict__ slopes,
                      const float* __restrict__ talk, const float* __restrict__ gate, long long gate_stride,
                      TO* __restrict__ out, long long o_stride, int T, int H, int G, int D, int page_size, float scale,
                      float eps, float mult, int window, int n_pages, int* err) {
  extern __shared__ __align__(16) float smem[];
  float* qs = smem;                           // [H][DQ]: the token's queries
  const int DQ = (D + 3) & ~3;
  float* ps = qs + H * DQ;                    // [H][32]: a tile's weights of every head
  float* ts = ps + H * 32;                    // [H][H]: the mixing matrix
  pdl_launch_dependents();
  const int t = blockIdx.x, h = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = h / (H / G);
  for (int i = threadIdx.x; i < H * H; i += blockDim.x) ts[i] = talk[i];
  const float slope = slopes[h];
  pdl_wait();
  const int pos = positions[t];
  const int req = token_req ? token_req[t] : t;
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int* bt = block_table + (size_t)req * bt_stride;
  for (int d = lane; d < DQ; d += 32) qs[h * DQ + d] = d < D ? q[(size_t)t * q_stride + (size_t)h * D + d] : 0.0f;
  __syncthreads();
  const float* qv = qs + h * DQ;
  const size_t head_rows = (size_t)c * page_size;
  auto key_row = [&](int p) -> const TC* {
    const int page = bt[p / page_size];
    if (!sglc_index_ok(page, n_pages, err)) return nullptr;
    return cache + (((size_t)page * G) * page_size + head_rows + (size_t)(p % page_size)) * D;
  };
  // first visit: this head's maximum and sum, a lane a key, merged over the lanes at the end
  float m = -INFINITY, l = 0.0f;
  for (int kt = lo / 32; kt <= pos / 32; kt++) {
    const int key = kt * 32 + lane;
    if (key < lo || key > pos) continue;
    const TC* kp = key_row(key);
    if (!kp) continue;
    const float s = talk_score(qv, kp, D, eps, scale, slope * (float)(pos - key));
    const float mn = fmaxf(m, s);
    l = l * expf(m - mn) + expf(s - mn);
    m = mn;
  }
  const float mh = warp_max(m);
  l = warp_sum(m == -INFINITY ? 0.0f : l * expf(m - mh));
  const float inv_l = 1.0f / l;
  // second visit: the weights themselves, mixed over the heads, applied to the values
  float acc[NV];
#pragma unroll
  for (int i = 0; i < NV; i++) acc[i] = 0.0f;
  for (int kt = lo / 32; kt <= pos / 32; kt++) {
    const int key0 = kt * 32, key = key0 + lane;
    float pw = 0.0f;
    if (key >= lo && key <= pos) {
      const TC* kp = key_row(key);
      if (kp) pw = expf(talk_score(qv, kp, D, eps, scale, slope * (float)(pos - key)) - mh) * inv_l;
    }
    __syncthreads();                          // everybody is done with the tile before
    ps[h * 32 + lane] = pw;
    __syncthreads();
    float mixed = 0.0f;
    for (int g = 0; g < H; g++) mixed = fmaf(ts[h * H + g], ps[g * 32 + lane], mixed);
    const int j1 = min(31, pos - key0);
    for (int j = max(0, lo - key0); j <= j1; j++) {
      const float w = __shfl_sync(0xffffffffu, mixed, j);
      const TC* vp = key_row(key0 + j);
      if (!vp) continue;
#pragma unroll
      for (int i = 0; i < NV; i++) {
        const int d = lane + 32 * i;
        if (d < D) acc[i] = fmaf(w, to_f32(vp[d]), acc[i]);
      }
    }
  }
  TO* op = out + (size_t)t * o_stride + (size_t)h * D;
  const float* gp = gate ? gate + (size_t)t * gate_stride + (size_t)h * D : nullptr;
#pragma unroll
  for (int i = 0; i < NV; i++) {
    const int d = lane + 32 * i;
    if (d < D) {
      float o = acc[i] * mult;
      if (gp) o *= 1.0f / (1.0f + expf(-gp[d]));
      op[d] = from_f32<TO>(o);
    }
  }
}

// x: float [T][H*D queries | G*D keys | ...] as projected; wq, wk: float [D]; q_out: float [T][H*D];
// cache: [n_pages][G][page_size][D] of cache_dtype; slots[t] = page * page_size + offset (negative: skip).
SGLC_API int sglc_talk_prep(const float* x, long long x_stride, const float* wq, const float* wk, float eps,
                            float* q_out, long long q_stride, void* cache, int cache_dtype, const int* slots, int T,
                            int H, int G, int D, int page_size, int n_pages, int* err, cudaStream_t stream) {
  if (T <= 0) return SGLC_OK;
  if (H <= 0 || G <= 0 || H % G != 0 || D <= 0 || page_size <= 0) return SGLC_ERR_ARGUMENT;
  if (cache_dtype == SGLC_F32)
    return sglc_launch(talk_prep_kernel<float>, dim3(T), dim3(TALK_PREP_WARPS * 32), 0, stream, 1, true, x, x_stride, wq,
                       wk, eps, q_out, q_stride, (float*)cache, slots, T, H, G, D, page_size, n_pages, err);
  if (cache_dtype == SGLC_BF16)
    return sglc_launch(talk_prep_kernel<__nv_bfloat16>, dim3(T), dim3(TALK_PREP_WARPS * 32), 0, stream, 1, true, x,
                       x_stride, wq, wk, eps, q_out, q_stride, (__nv_bfloat16*)cache, slots, T, H, G, D, page_size,
                       n_pages, err);
  return SGLC_ERR_ARGUMENT;
}

// q: float [T][H*D] from sglc_talk_prep; slopes: float [H]; talk: float [H][H]; gate: float rows
// [T][H*D] (null: no gate); out: [T][H*D] of out_dtype; token_req null: token t is request t.
SGLC_API int sglc_talk_attention(const float* q, long long q_stride, const void* cache, int cache_dtype,
                                 const int* block_table, int bt_stride, const int* token_req, const int* positions,
                                 const float* slopes, const float* talk, const float* gate, long long gate_stride,
                                 void* out, long long o_stride, int out_dtype, int T, int H, int G, int D,
                                 int page_size, float scale, float eps, float mult, int window, int n_pages, int* err,
                                 cudaStream_t stream) {
  if (T <= 0) return SGLC_OK;
  if (H <= 0 || G <= 0 || H % G != 0 || D <= 0 || page_size <= 0 || window < 0) return SGLC_ERR_ARGUMENT;
  if (H > TALK_MAX_HEADS || D > TALK_MAX_DIM) return SGLC_ERR_UNSUPPORTED;
  // (rows are read four elements a load where the head size allows: q rows are padded to that)
  const size_t smem = ((size_t)H * ((D + 3) & ~3) + (size_t)H * 32 + (size_t)H * H) * sizeof(float);
  const int nv = (D + 31) / 32;
#define TALK_GO(TC, TO, NV)                                                                                        \
  do {                                                                                                             \
    if (smem > 48 * 1024)                                                                                          \
      cudaFuncSetAttribute(talk_attention_kernel<TC, TO, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    return sglc_launch(talk_attention_kernel<TC, TO, NV>, dim3(T), dim3(H * 32), smem, stream, 1, true, q, q_stride, \
                       (const TC*)cache, block_table, bt_stride, token_req, positions, slopes, talk, gate,         \
                       gate_stride, (TO*)out, o_stride, T, H, G, D, page_size, scale, eps, mult, window, n_pages,  \
                       err);                                                                                       \
  } while (0)
#define TALK_NV(TC, TO)                     \
  do {                                      \
    if (nv <= 1) TALK_GO(TC, TO, 1);        \
    if (nv <= 2) TALK_GO(TC, TO, 2);        \
    if (nv <= 4) TALK_GO(TC, TO, 4);        \
    TALK_GO(TC, TO, 8);                     \
  } while (0)
  if (cache_dtype == SGLC_F32 && out_dtype == SGLC_F32) TALK_NV(float, float);
  if (cache_dtype == SGLC_BF16 && out_dtype == SGLC_BF16) TALK_NV(__nv_bfloat16, __nv_bfloat16);
#undef TALK_NV
#undef TALK_GO
  return SGLC_ERR_ARGUMENT;
}
