// Causal attention over the paged cache for any mix of prompt portions and single decoded
// tokens.  All arithmetic is 32-bit:
//   s[p] = (q·K_p)*scale for the keys p the query may see (p <= its position,
//   and p > position - window if a window is set); m = max s; e = exp(s-m);
//   o = sum_p e[p]*V_p / sum_p e[p]
// (reference src/gpt2.c:238-270; GPU twin k_attn, src/cuda_backend.cu:1600-1651).
// A (token, head) is one warp.  It takes its keys in tiles of 32 by absolute position (tile k
// holds positions 32k..32k+31: a lane a key for the scores, the softmax statistics kept online
// from tile to tile, then a lane per output dimension over the tile's values), so its order of
// additions depends only on its own first and last visible key, never on the rest of the batch:
// the result is the same, bit for bit, however the tokens were cut into steps.  The tokens of a
// block that belong to one request share each tile of that request's keys and values in shared
// memory (a block of eight consecutive tokens of a prompt portion reads them once instead of
// eight times: the reference's kernel, one block per token, reads them per token).  This is the
// kernel of the 32-bit path and the general fallback of the bfloat16 path.
#include "common.cuh"

SGLC_DEFINE_ERROR_STRING()

// Four consecutive cache elements as 32-bit floats, by one load (p is aligned to four elements).
__device__ __forceinline__ void load4(const float* p, float* v) {
  const float4 x = *reinterpret_cast<const float4*>(p);
  v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float* v) {
  const uint2 x = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&x.x);
  const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&x.y);
  v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
}

// W: tokens of a block (a warp each).  Threads beyond the tokens' warps only help to stage tiles.
// EXT: the form with a value size DV of its own (a page then holds Hkv x page_size x D keys
// followed by Hkv x page_size x DV values), a chunk mask (a query sees only keys of its own chunk of
// `chunk` positions, counted from position 0) and a sink per head (a learned score that joins the
// softmax's denominator once, with no key and no value).  Without EXT the three arguments are unused.
template <typename TQ, typename TC, typename TO, int W, int THREADS, bool EXT>
__global__ void __launch_bounds__(THREADS, THREADS == 256 ? 3 : 4)     // (registers capped so that three blocks of 256 share an SM)
attention_simt_kernel(const TQ* __restrict__ q, int q_stride, const TC* __restrict__ cache,
                      const int* __restrict__ block_table, int bt_stride,
                      const int* __restrict__ token_req, const int* __restrict__ positions,
                      TO* __restrict__ out, int o_stride, int T, int H, int Hkv, int D, int page_size,
                      float scale, int window, int n_pages, int* err, int kv_shared,
                      int DV_arg, int chunk, const float* __restrict__ sinks, int n_splits,
                      float* __restrict__ part_ws, int head_rows) {
  const int DV = EXT ? DV_arg : D;
  // head_rows (EXT, a step of single tokens): the block's warps are the query heads that share one
  // key/value head, all of ONE token (blockIdx.x), instead of consecutive tokens of one head: the
  // tile of keys and values is staged once for all of them
  const bool hrows = EXT && head_rows;
  const int grp = H / Hkv;
  extern __shared__ __align__(16) float smem[];
  __shared__ int s_req[W], s_lo[W], s_pos[W];
  // padded key rows: a lane a key without bank conflicts (by 4 where rows are read 16 bytes at a time)
  const bool wide = D % 4 == 0;
  const int DP = wide ? D + 4 : D + 1;
  float* Ks = smem;                           // [32][DP]
  float* Vs = Ks + 32 * DP;                   // [32][D]
  float* pw = Vs + 32 * DV;                   // [W][32]: a tile's weights (16-byte aligned whatever D is)
  float* qs = pw + W * 32;                    // [W][D]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int hk = hrows ? (int)blockIdx.y : (int)blockIdx.y / grp;
  const int h = hrows ? hk * grp + min(warp, grp - 1) : (int)blockIdx.y;      // this warp's query head
  const int t0 = hrows ? (int)blockIdx.x : (int)blockIdx.x * W;
  const int my_t = hrows ? t0 : t0 + warp;                                     // this warp's token
  if (tid < W) {
    const int t = hrows ? t0 : t0 + tid;
    const bool on = hrows ? tid < grp : t < T;
    const int pos = on ? positions[t] : -1;
    s_req[tid] = on ? token_req[t] : -1;
    s_pos[tid] = pos;
    int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    if (EXT && chunk > 0 && pos >= 0) lo = max(lo, pos / chunk * chunk);
    s_lo[tid] = lo;
  }
  const bool mine = warp < W && (hrows ? warp < grp : t0 + warp < T);
  if (mine) {
    const TQ* qp = q + (size_t)my_t * q_stride + (size_t)h * D;
    for (int d = lane; d < D; d += 32) qs[warp * D + d] = to_f32(qp[d]);
  }
  __syncthreads();
  const int my_req = mine ? s_req[warp] : -2, my_lo = mine ? s_lo[warp] : 0, my_pos = mine ? s_pos[warp] : -1;
  float m = -INFINITY, l = 0.0f;
  float acc[8];                               // dims lane, lane + 32, ... of the output
#pragma unroll
  for (int i = 0; i < 8; i++) acc[i] = 0.0f;
  // kv_shared: a page holds one block of rows that are keys and values at once (a latent)
  const size_t page_elems = EXT ? (size_t)Hkv * page_size * (D + DV) : (size_t)(kv_shared ? 1 : 2) * Hkv * page_size * D;
  const size_t head_off = (size_t)hk * page_size * D, v_off = kv_shared ? 0 : (size_t)Hkv * page_size * D;

  // The tokens of a block that belong to one request (a run: a request's tokens lie together)
  // share the tiles of that request's keys and values; the runs of a block take turns.
  for (int lead = 0; lead < W; lead++) {
    const int rl = s_req[lead];
    if (rl < 0 || (lead > 0 && s_req[lead - 1] == rl)) continue;         // not the start of a run
    int lo_min = s_lo[lead], pos_max = s_pos[lead];
    for (int w = lead + 1; w < W && s_req[w] == rl; w++) {
      lo_min = min(lo_min, s_lo[w]);
      pos_max = max(pos_max, s_pos[w]);
    }
    const int* bt = block_table + (size_t)rl * bt_stride;
    int kt_first = lo_min / 32, kt_end = pos_max / 32 + 1;
    if (EXT && part_ws) {
      // the keys in sight dealt to the blocks of grid.z in runs of whole tiles (a step of single
      // tokens: a block has one token, so the run follows from its own first and last key)
      const int per = (kt_end - kt_first + n_splits - 1) / n_splits;
      kt_first += (int)blockIdx.z * per;
      kt_end = min(kt_end, kt_first + per);
    }
    for (int kt = kt_first; kt < kt_end; kt++) {
      const int key0 = kt * 32;
      __syncthreads();                        // the tile before has been used by everybody
      {
        // THREADS/32 threads bring one key and its value: the page is looked up once a key, and a
        // thread's loads do not depend on one another
        constexpr int TPK = THREADS / 32;
        const int j = tid / TPK, part = tid % TPK, p = key0 + j;
        const TC* kp = nullptr;
        if (p >= lo_min && p <= pos_max) {
          const int page = bt[p / page_size];
          if (sglc_index_ok(page, n_pages, err))
            kp = cache + (size_t)page * page_elems + head_off + (size_t)(p % page_size) * D;
        }
        if (EXT) {
          const TC* vp = kp ? cache + (size_t)(bt[p / page_size]) * page_elems + (size_t)Hkv * page_size * D +
                                  ((size_t)hk * page_size + p % page_size) * DV
                            : nullptr;
          if (D % 4 == 0 && DV % 4 == 0) {      // (rows, pages and both blocks of a page start at multiples of four)
            for (int d = part * 4; d < D; d += 4 * TPK) {
              float k4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
              if (kp) load4(kp + d, k4);
              *reinterpret_cast<float4*>(&Ks[j * DP + d]) = make_float4(k4[0], k4[1], k4[2], k4[3]);
            }
            for (int d = part * 4; d < DV; d += 4 * TPK) {
              float v4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
              if (vp) load4(vp + d, v4);
              *reinterpret_cast<float4*>(&Vs[j * DV + d]) = make_float4(v4[0], v4[1], v4[2], v4[3]);
            }
          } else {
            for (int d = part; d < D; d += TPK) Ks[j * DP + d] = kp ? to_f32(kp[d]) : 0.0f;
            for (int d = part; d < DV; d += TPK) Vs[j * DV + d] = vp ? to_f32(vp[d]) : 0.0f;
          }
        } else if (D % 4 == 0) {
          for (int d = part * 4; d < D; d += 4 * TPK) {
            float k4[4] = {0.0f, 0.0f, 0.0f, 0.0f}, v4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            if (kp) {
              load4(kp + d, k4);
              load4(kp + v_off + d, v4);
            }
            *reinterpret_cast<float4*>(&Ks[j * DP + d]) = make_float4(k4[0], k4[1], k4[2], k4[3]);
            *reinterpret_cast<float4*>(&Vs[j * D + d]) = make_float4(v4[0], v4[1], v4[2], v4[3]);
          }
        } else {
          for (int d = part; d < D; d += TPK) {
            Ks[j * DP + d] = kp ? to_f32(kp[d]) : 0.0f;
            Vs[j * D + d] = kp ? to_f32(kp[v_off + d]) : 0.0f;
          }
        }
      }
      __syncthreads();
      // a token takes the tile if it belongs to the run and the tile holds keys it may see
      if (my_req == rl && key0 <= my_pos && key0 + 31 >= my_lo) {
        const int key = key0 + lane;
        const bool valid = key >= my_lo && key <= my_pos;
        const float* qv = qs + warp * D;
        const float* kr = Ks + lane * DP;
        float sc = 0.0f;
        if (wide) {                           // (the same additions in the same order, four a load)
          for (int d = 0; d < D; d += 4) {
            const float4 q4 = *reinterpret_cast<const float4*>(qv + d);
            const float4 k4 = *reinterpret_cast<const float4*>(kr + d);
            sc = fmaf(q4.x, k4.x, sc);
            sc = fmaf(q4.y, k4.y, sc);
            sc = fmaf(q4.z, k4.z, sc);
            sc = fmaf(q4.w, k4.w, sc);
          }
        } else {
          for (int d = 0; d < D; d++) sc = fmaf(qv[d], kr[d], sc);
        }
        sc = valid ? sc * scale : -INFINITY;
        const float m_new = fmaxf(m, warp_max(sc));
        const float corr = expf(m - m_new);                             // (first tile: exp(-inf) = 0)
        const float p = valid ? expf(sc - m_new) : 0.0f;
        l = l * corr + warp_sum(p);
        m = m_new;
        pw[warp * 32 + lane] = p;
        __syncwarp();
        float pj[32];                         // the tile's weights, read once for all output columns
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          const float4 p4 = *reinterpret_cast<const float4*>(&pw[warp * 32 + j]);
          pj[j] = p4.x; pj[j + 1] = p4.y; pj[j + 2] = p4.z; pj[j + 3] = p4.w;
        }
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const int d = lane + 32 * i;
          if (d < DV) {
            float a = acc[i] * corr;
#pragma unroll
            for (int j = 0; j < 32; j++) a = fmaf(pj[j], Vs[j * DV + d], a);
            acc[i] = a;
          }
        }
        __syncwarp();
      }
    }
  }
  if (EXT && part_ws) {
    // this block's share of the keys: maximum, sum and unnormalised result, for the merge
    if (mine) {
      float* rec = part_ws + (((size_t)my_t * H + h) * n_splits + blockIdx.z) * (DV + 2);
      if (lane == 0) { rec[0] = m; rec[1] = l; }
#pragma unroll
      for (int i = 0; i < 8; i++) {
        const int d = lane + 32 * i;
        if (d < DV) rec[2 + d] = acc[i];
      }
    }
    return;
  }
  if (mine) {
    TO* op = out + (size_t)my_t * o_stride + (size_t)h * DV;
    float inv = 1.0f / l;
    if (EXT && sinks) {                        // the sink joins the denominator: exp(sink - max) once
      const float sk = sinks[h], m_all = fmaxf(m, sk);
      inv = expf(m - m_all) / (l * expf(m - m_all) + expf(sk - m_all));
    }
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const int d = lane + 32 * i;
      if (d < DV) op[d] = from_f32<TO>(acc[i] * inv);
    }
  }
}

// q: first query element of token 0 (rows q_stride apart, heads side by side); cache: one
// layer's pages; block_table: [n_requests][bt_stride] page ids; token_req[t]: row of the
// block table for token t; positions[t]: absolute position of token t (its own key is the
// last one it sees); out: [T][o_stride].  max_keys: the most keys any token of this launch
// sees.  q/out dtype = act_dtype, cache dtype = cache_dtype.  n_pages and err serve the
// bounds-check build (page ids are compared with n_pages; err gets the flag).  max_q_len: the
// longest portion of the step (1: every request brings one token, and a block takes one token).
static int attention_simt_run(const void* q, int q_stride, const void* cache,
                              const int* block_table, int bt_stride, const int* token_req,
                              const int* positions, void* out, int o_stride, int T, int H,
                              int Hkv, int D, int page_size, float scale, int window,
                              int max_keys, int act_dtype, int cache_dtype, int n_pages, int* err,
                              int max_q_len, int kv_shared, cudaStream_t stream, bool ext = false, int DV = 0,
                              int chunk = 0, const float* sinks = nullptr, int n_splits = 1, float* part_ws = nullptr) {
  if (T <= 0) return SGLC_OK;
  if (!ext) DV = D;
  if (DV <= 0 || DV > 256 || chunk < 0) return ext ? SGLC_ERR_UNSUPPORTED : SGLC_ERR_ARGUMENT;
  if (H <= 0 || Hkv <= 0 || H % Hkv != 0 || D <= 0 || page_size <= 0 || max_keys <= 0)
    return SGLC_ERR_ARGUMENT;
  if (H > 65535 || D > 256) return SGLC_ERR_UNSUPPORTED;
  // single tokens of many requests share nothing: a token a block; portions: eight tokens a block
  const bool single = max_q_len <= 1;
  const int W = single ? 1 : 8;
  const size_t smem = ((size_t)32 * (D % 4 == 0 ? D + 4 : D + 1) + (size_t)32 * DV + (size_t)W * D + (size_t)W * 32) * sizeof(float);
  if (part_ws && (!ext || !single || n_splits < 1 || n_splits > 65535)) return SGLC_ERR_ARGUMENT;
  dim3 grid((T + W - 1) / W, H, part_ws ? n_splits : 1);
  // single tokens whose shares are merged afterwards: where 2 to 8 query heads share a key/value
  // head, a block takes them all (the eight-warp form, its warps being heads of one token)
  const int head_rows = (part_ws && H / Hkv >= 2 && H / Hkv <= 8) ? 1 : 0;
  const size_t smem_rows = ((size_t)32 * (D % 4 == 0 ? D + 4 : D + 1) + (size_t)32 * DV + (size_t)8 * D + (size_t)8 * 32) * sizeof(float);
  if (head_rows) {
    const dim3 grid_rows(T, Hkv, n_splits);
#define LAUNCH_R(TQ, TC, TO)                                                                            \
  do {                                                                                                 \
    if (smem_rows > 48 * 1024)                                                                         \
      cudaFuncSetAttribute(attention_simt_kernel<TQ, TC, TO, 8, 256, true>,                            \
                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_rows);               \
    attention_simt_kernel<TQ, TC, TO, 8, 256, true><<<grid_rows, 256, smem_rows, stream>>>(            \
        (const TQ*)q, q_stride, (const TC*)cache, block_table, bt_stride, token_req, positions,        \
        (TO*)out, o_stride, T, H, Hkv, D, page_size, scale, window, n_pages, err, kv_shared, DV,       \
        chunk, sinks, n_splits, part_ws, 1);                                                           \
  } while (0)
    if (act_dtype == SGLC_F32 && cache_dtype == SGLC_F32) LAUNCH_R(float, float, float);
    else if (act_dtype == SGLC_BF16 && cache_dtype == SGLC_BF16) LAUNCH_R(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
    else return SGLC_ERR_ARGUMENT;
#undef LAUNCH_R
    return sglc_launch_status();
  }
#define LAUNCH_E(TQ, TC, TO, WW, TH, EX)                                                               \
  do {                                                                                                 \
    if (smem > 48 * 1024)                                                                              \
      cudaFuncSetAttribute(attention_simt_kernel<TQ, TC, TO, WW, TH, EX>,                              \
                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                    \
    attention_simt_kernel<TQ, TC, TO, WW, TH, EX><<<grid, TH, smem, stream>>>(                          \
        (const TQ*)q, q_stride, (const TC*)cache, block_table, bt_stride, token_req, positions,        \
        (TO*)out, o_stride, T, H, Hkv, D, page_size, scale, window, n_pages, err, kv_shared, DV,       \
        chunk, sinks, n_splits, part_ws, 0);                                                           \
  } while (0)
#define LAUNCH(TQ, TC, TO, WW, TH)                                                                     \
  do {                                                                                                 \
    if (ext) LAUNCH_E(TQ, TC, TO, WW, TH, true);                                                       \
    else LAUNCH_E(TQ, TC, TO, WW, TH, false);                                                          \
  } while (0)
  if (act_dtype == SGLC_F32 && cache_dtype == SGLC_F32) {
    if (single) LAUNCH(float, float, float, 1, 128);
    else LAUNCH(float, float, float, 8, 256);
  } else if (act_dtype == SGLC_BF16 && cache_dtype == SGLC_BF16) {
    if (single) LAUNCH(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16, 1, 128);
    else LAUNCH(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16, 8, 256);
  } else {
    return SGLC_ERR_ARGUMENT;
  }
#undef LAUNCH
#undef LAUNCH_E
  return sglc_launch_status();
}

SGLC_API int sglc_attention_simt(const void* q, int q_stride, const void* cache,
                                 const int* block_table, int bt_stride, const int* token_req,
                                 const int* positions, void* out, int o_stride, int T, int H,
                                 int Hkv, int D, int page_size, float scale, int window,
                                 int max_keys, int act_dtype, int cache_dtype, int n_pages, int* err,
                                 int max_q_len, cudaStream_t stream) {
  return attention_simt_run(q, q_stride, cache, block_table, bt_stride, token_req, positions, out, o_stride,
                            T, H, Hkv, D, page_size, scale, window, max_keys, act_dtype, cache_dtype,
                            n_pages, err, max_q_len, 0, stream);
}

// The same over a cache whose pages hold one block of rows [Hkv][page_size][D] that serve as keys
// and as values (attention over a latent that both are read from): cache [n_pages][1][Hkv][page_size][D].
SGLC_API int sglc_attention_simt_shared(const void* q, int q_stride, const void* cache,
                                        const int* block_table, int bt_stride, const int* token_req,
                                        const int* positions, void* out, int o_stride, int T, int H,
                                        int Hkv, int D, int page_size, float scale, int window,
                                        int max_keys, int act_dtype, int cache_dtype, int n_pages, int* err,
                                        int max_q_len, cudaStream_t stream) {
  return attention_simt_run(q, q_stride, cache, block_table, bt_stride, token_req, positions, out, o_stride,
                            T, H, Hkv, D, page_size, scale, window, max_keys, act_dtype, cache_dtype,
                            n_pages, err, max_q_len, 1, stream);
}

// The extended form: values of size DV beside keys of size D (cache [n_pages][Hkv x page_size x D keys |
// Hkv x page_size x DV values]; out rows hold H heads of DV), `chunk` > 0: a query sees the keys of its
// own chunk of so many positions only; `sinks` (float [H] or null): a score per head that joins the
// softmax's denominator.
SGLC_API int sglc_attention_simt_ext(const void* q, int q_stride, const void* cache,
                                     const int* block_table, int bt_stride, const int* token_req,
                                     const int* positions, void* out, int o_stride, int T, int H,
                                     int Hkv, int D, int DV, int page_size, float scale, int window, int chunk,
                                     const float* sinks, int max_keys, int act_dtype, int cache_dtype, int n_pages,
                                     int* err, int max_q_len, cudaStream_t stream) {
  return attention_simt_run(q, q_stride, cache, block_table, bt_stride, token_req, positions, out, o_stride,
                            T, H, Hkv, D, page_size, scale, window, max_keys, act_dtype, cache_dtype,
                            n_pages, err, max_q_len, 0, stream, true, DV, chunk, sinks);
}

// The merge behind a launch that dealt a token's keys to several blocks (a step of single tokens):
// the shares' maxima, sums and unnormalised results [T][H][n_splits][DV + 2] become the head's
// result, the sink (if any) joining the denominator once.  A warp a (token, head).
template <typename TO>
__global__ void __launch_bounds__(128)
attention_merge_kernel(const float* __restrict__ part_ws, int n_splits, const float* __restrict__ sinks,
                       TO* __restrict__ out, int o_stride, int T, int H, int DV) {
  pdl_launch_dependents();
  const long long item = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  pdl_wait();
  if (item >= (long long)T * H) return;
  const int t = (int)(item / H), h = (int)(item % H);
  const float* rec = part_ws + (size_t)item * n_splits * (DV + 2);
  float M = sinks ? sinks[h] : -INFINITY;
  for (int s = 0; s < n_splits; s++)
    if (rec[(size_t)s * (DV + 2) + 1] > 0.0f) M = fmaxf(M, rec[(size_t)s * (DV + 2)]);
  float L = sinks ? expf(sinks[h] - M) : 0.0f;
  for (int s = 0; s < n_splits; s++) {
    const float ls = rec[(size_t)s * (DV + 2) + 1];
    if (ls > 0.0f) L += ls * expf(rec[(size_t)s * (DV + 2)] - M);
  }
  const float inv = 1.0f / L;
  TO* op = out + (size_t)t * o_stride + (size_t)h * DV;
  for (int d = lane; d < DV; d += 32) {
    float o = 0.0f;
    for (int s = 0; s < n_splits; s++)
      if (rec[(size_t)s * (DV + 2) + 1] > 0.0f) o += rec[(size_t)s * (DV + 2) + 2 + d] * expf(rec[(size_t)s * (DV + 2)] - M);
    op[d] = from_f32<TO>(o * inv);
  }
}

// The extended form for a step of single tokens with each token's keys dealt to n_splits blocks:
// part_ws holds T x H x n_splits x (DV + 2) floats; two launches (the shares, then the merge).
SGLC_API int sglc_attention_simt_ext_split(const void* q, int q_stride, const void* cache,
                                           const int* block_table, int bt_stride, const int* token_req,
                                           const int* positions, void* out, int o_stride, int T, int H,
                                           int Hkv, int D, int DV, int page_size, float scale, int window, int chunk,
                                           const float* sinks, int max_keys, int act_dtype, int cache_dtype,
                                           int n_pages, int* err, int n_splits, float* part_ws, cudaStream_t stream) {
  if (T <= 0) return SGLC_OK;
  if (!part_ws || n_splits < 1) return SGLC_ERR_ARGUMENT;
  const int code = attention_simt_run(q, q_stride, cache, block_table, bt_stride, token_req, positions, out, o_stride,
                                      T, H, Hkv, D, page_size, scale, window, max_keys, act_dtype, cache_dtype,
                                      n_pages, err, 1, 0, stream, true, DV, chunk, nullptr, n_splits, part_ws);
  if (code != SGLC_OK) return code;
  const dim3 grid((unsigned)(((long long)T * H + 3) / 4));
  if (act_dtype == SGLC_F32)
    return sglc_launch(attention_merge_kernel<float>, grid, dim3(128), 0, stream, 1, true, (const float*)part_ws,
                       n_splits, sinks, (float*)out, o_stride, T, H, DV);
  return sglc_launch(attention_merge_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, 1, true,
                     (const float*)part_ws, n_splits, sinks, (__nv_bfloat16*)out, o_stride, T, H, DV);
}
