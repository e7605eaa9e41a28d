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

// ---------------------------------------------------------------------------------------------
// The same attention in tiles on the tensor cores (bfloat16 cache): a block takes 16 consecutive
// queries of one request and all heads, a warp a head.  Keys come 32 at a time by absolute position
// into shared memory, all key heads of them, 16 bytes a cp.async, the next tile on its way while one
// is worked on.  S = Q K^T by mma.sync m16n8k16 (bfloat16 operands, 32-bit sums; a 32-bit query
// enters as two operands, its bfloat16 rounding and what that left; the key's 1/rms, taken from
// the staged rows, the scale and the distance penalty are applied to the accumulator).
// First all tiles for every row's maximum and sum; then all tiles again: p = exp(s - max) / sum in
// 32-bit, exchanged between the warps through shared memory, mixed (32-bit), packed to bfloat16 as
// the A operand of O += P' V, whose B operand is the same staged tile read transposed.
constexpr int TT_ROWS = 16;
constexpr int TT_KEYS = 32;
constexpr int TT_PPITCH = 40;       // floats between rows of a head's weights: 8-byte reads without conflicts
constexpr int TT_MAX_HEADS = 16;

__device__ __forceinline__ void tt_ldsm4(uint32_t addr, uint32_t* r) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void tt_ldsm4_t(uint32_t addr, uint32_t* r) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void tt_mma(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t tt_pack(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ void tt_cp16(uint32_t dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;       // no source bytes: the 16 destination bytes are zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ float tt_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Blocks of one grid.z column form a cluster and share a tile's keys between them (below).
__device__ __forceinline__ uint32_t tt_peer(const void* local, uint32_t rank) {
  uint32_t raddr;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(raddr) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
  return raddr;
}
__device__ __forceinline__ float2 tt_peer_ld2(uint32_t raddr) {
  float2 v;
  asm volatile("ld.shared::cluster.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(raddr) : "memory");
  return v;
}
__device__ __forceinline__ void tt_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// gridDim.z = S blocks (a cluster, S > 1) divide the key tiles of one tile of queries: each visits
// its share for the maxima and sums, the S pairs per (head, row) are merged through the cluster's
// shared memory, each forms mixed weights and a partial result over its share, and block 0 adds
// the partial results (the result is linear in the normalised weights) and writes.  This is the
// form for few tiles of queries (decoding), where one block a request leaves the GPU idle.
template <int ND16>      // head size / 16
__global__ void __launch_bounds__(TT_MAX_HEADS * 32)
talk_tiles_kernel(const float* __restrict__ q, long long q_stride, const __nv_bfloat16* __restrict__ cache,
                  const int* __restrict__ block_table, int bt_stride, const int* __restrict__ q_start,
                  const int* __restrict__ kv_len, const float* __restrict__ slopes, const float* __restrict__ talk,
                  const float* __restrict__ gate, long long gate_stride, __nv_bfloat16* __restrict__ out,
                  long long o_stride, int H, int G, int page_size, float scale, float eps, float mult, int window,
                  int nbuf, int n_pages, int* err) {
  constexpr int D = ND16 * 16, DP = D + 8, CH = D / 8;
  extern __shared__ __align__(16) unsigned char tt_smem[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(tt_smem);            // [2][H][16][DP]: q = high + low part
  __nv_bfloat16* Ks = Qs + (size_t)2 * H * TT_ROWS * DP;                    // [nbuf][G][32][DP]
  float* kinv = reinterpret_cast<float*>(Ks + (size_t)nbuf * G * TT_KEYS * DP);   // [nbuf][G][32]
  float* Ps = kinv + (size_t)nbuf * G * TT_KEYS;                                          // [H][16][TT_PPITCH]
  float* Ts = Ps + (size_t)H * TT_ROWS * TT_PPITCH;                         // [H][H]
  float* stat = Ts + ((H * H + 1) & ~1);                                    // [H][16][2]: (max, sum), S > 1
  float* Os = stat + (size_t)H * TT_ROWS * 2;                               // [H][rows][D]: partial result, S > 1
  const int S = gridDim.z, z = blockIdx.z;
  pdl_launch_dependents();
  const int tid = threadIdx.x, h = tid >> 5, lane = tid & 31, nthr = blockDim.x;
  const int c = h / (H / G);
  for (int i = tid; i < H * H; i += nthr) Ts[i] = talk[i];
  constexpr float LOG2E = 1.4426950408889634f;
  const float slope2 = slopes[h] * LOG2E, scale2 = scale * LOG2E;
  pdl_wait();
  const int r = blockIdx.y;
  const int t0 = q_start[r], n = q_start[r + 1] - t0, row0 = blockIdx.x * TT_ROWS;
  if (row0 >= n) return;
  const int rows = min(TT_ROWS, n - row0);
  const int base_pos = kv_len[r] - n + row0, p_last = base_pos + rows - 1;
  const int lo_blk = (window > 0 && base_pos - window + 1 > 0) ? base_pos - window + 1 : 0;
  const int* bt = block_table + (size_t)r * bt_stride;
  // the tile's queries, to bfloat16
  for (int i = tid; i < H * TT_ROWS * (D / 4); i += nthr) {
    const int d4 = i % (D / 4), row = (i / (D / 4)) % TT_ROWS, hh = i / (D / 4 * TT_ROWS);
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (row < rows) v = *reinterpret_cast<const float4*>(q + (size_t)(t0 + row0 + row) * q_stride + (size_t)hh * D + d4 * 4);
    // a 32-bit query as two bfloat16 operands: what the first leaves, the second takes
    const float e[4] = {v.x, v.y, v.z, v.w};
    float lo[4];
#pragma unroll
    for (int k = 0; k < 4; k++) lo[k] = e[k] - __bfloat162float(__float2bfloat16_rn(e[k]));
    uint2 w, wl;
    w.x = tt_pack(e[0], e[1]);
    w.y = tt_pack(e[2], e[3]);
    wl.x = tt_pack(lo[0], lo[1]);
    wl.y = tt_pack(lo[2], lo[3]);
    __nv_bfloat16* dst = Qs + ((size_t)hh * TT_ROWS + row) * DP + d4 * 4;
    *reinterpret_cast<uint2*>(dst) = w;
    *reinterpret_cast<uint2*>(dst + (size_t)H * TT_ROWS * DP) = wl;
  }
  // this block's share of the key tiles (none, where there are fewer tiles than blocks)
  const int kt_all = lo_blk / TT_KEYS, nt_all = p_last / TT_KEYS - kt_all + 1;
  const int kt_lo = kt_all + nt_all * z / S, NT = kt_all + nt_all * (z + 1) / S - kt_lo, total = 2 * NT;
  const uint32_t ks_base = (uint32_t)__cvta_generic_to_shared(Ks);
  auto issue = [&](int it, int buf) {
    const int key0 = (kt_lo + it % NT) * TT_KEYS;
    const uint32_t dst0 = ks_base + (uint32_t)buf * G * TT_KEYS * DP * 2;
    for (int i = tid; i < G * TT_KEYS * CH; i += nthr) {
      const int ch = i % CH, kl = (i / CH) % TT_KEYS, g = i / (CH * TT_KEYS);
      const int j = key0 + kl;
      bool valid = j >= lo_blk && j <= p_last;
      const __nv_bfloat16* src = cache;
      if (valid) {
        const int page = bt[j / page_size];
        valid = sglc_index_ok(page, n_pages, err);
        if (valid) src = cache + (((size_t)page * G + g) * page_size + (size_t)(j % page_size)) * D + ch * 8;
      }
      tt_cp16(dst0 + (uint32_t)((g * TT_KEYS + kl) * DP + ch * 8) * 2, src, valid);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  const int g4 = lane >> 2, c2 = (lane & 3) * 2;
  const int pos0 = base_pos + g4, pos1 = pos0 + 8;
  const bool ok0 = g4 < rows, ok1 = g4 + 8 < rows;
  const uint32_t q_addr = (uint32_t)__cvta_generic_to_shared(Qs) +
                          (uint32_t)(((h * TT_ROWS + (lane & 15)) * DP + (lane >> 4) * 8) * 2);
  const uint32_t q_low = (uint32_t)(H * TT_ROWS * DP * 2);
  // B of S: lane -> key (lane / 16) * 8 + lane % 8 of a pair of key octets, columns ((lane / 8) % 2) * 8
  const uint32_t kb_off = (uint32_t)(((c * TT_KEYS + (lane >> 4) * 8 + (lane & 7)) * DP + ((lane >> 3) & 1) * 8) * 2);
  // B of O (transposed read): lane -> key ((lane / 8) % 2) * 8 + lane % 8 of 16, columns (lane / 16) * 8
  const uint32_t vb_off = (uint32_t)(((c * TT_KEYS + ((lane >> 3) & 1) * 8 + (lane & 7)) * DP + (lane >> 4) * 8) * 2);
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f, il0 = 0.f, il1 = 0.f;
  float o[2 * ND16][4];
#pragma unroll
  for (int i = 0; i < 2 * ND16; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  // every key's 1/rms of `count` staged tiles from buffer `first` on
  auto norms = [&](int first, int count) {
    const __nv_bfloat16* kt_rows = Ks + (size_t)first * G * TT_KEYS * DP;
    for (int i = tid; i < count * G * TT_KEYS; i += nthr) {
      const uint4* row = reinterpret_cast<const uint4*>(kt_rows + (size_t)i * DP);
      float ss = 0.f;
#pragma unroll
      for (int ch = 0; ch < CH; ch++) {
        const uint4 v = row[ch];
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; e++) {
          const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&w[e]);
          const float x = __low2float(b), y = __high2float(b);
          ss = fmaf(x, x, ss);
          ss = fmaf(y, y, ss);
        }
      }
      kinv[first * G * TT_KEYS + i] = 1.0f / sqrtf(ss / (float)D + eps);
    }
  };
  // after the first visit: the rows' maxima and sums over the four threads that share a row, and
  // over the blocks of the cluster
  auto finish_first = [&]() {
#pragma unroll
    for (int hf = 0; hf < 2; hf++) {
      float mx = hf ? m1 : m0, l = hf ? l1 : l0;
      float ma = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      ma = fmaxf(ma, __shfl_xor_sync(0xffffffffu, ma, 2));
      l = mx > -INFINITY ? l * tt_exp2(mx - ma) : 0.f;
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      if (hf) { m1 = ma; l1 = l; } else { m0 = ma; l0 = l; }
    }
    if (S > 1) {
      if ((lane & 3) == 0) {
        *reinterpret_cast<float2*>(stat + (h * TT_ROWS + g4) * 2) = make_float2(m0, l0);
        *reinterpret_cast<float2*>(stat + (h * TT_ROWS + g4 + 8) * 2) = make_float2(m1, l1);
      }
      tt_cluster_sync();
      float ma0 = -INFINITY, ma1 = -INFINITY;
      for (int zz = 0; zz < S; zz++) {
        ma0 = fmaxf(ma0, tt_peer_ld2(tt_peer(stat + (h * TT_ROWS + g4) * 2, zz)).x);
        ma1 = fmaxf(ma1, tt_peer_ld2(tt_peer(stat + (h * TT_ROWS + g4 + 8) * 2, zz)).x);
      }
      float s0 = 0.f, s1 = 0.f;
      for (int zz = 0; zz < S; zz++) {
        const float2 a = tt_peer_ld2(tt_peer(stat + (h * TT_ROWS + g4) * 2, zz));
        const float2 b = tt_peer_ld2(tt_peer(stat + (h * TT_ROWS + g4 + 8) * 2, zz));
        if (a.x > -INFINITY) s0 = fmaf(a.y, tt_exp2(a.x - ma0), s0);
        if (b.x > -INFINITY) s1 = fmaf(b.y, tt_exp2(b.x - ma1), s1);
      }
      m0 = ma0; l0 = s0; m1 = ma1; l1 = s1;
    }
    il0 = l0 > 0.f ? 1.0f / l0 : 0.f;
    il1 = l1 > 0.f ? 1.0f / l1 : 0.f;
    if (!(m0 > -INFINITY)) m0 = 0.f;
    if (!(m1 > -INFINITY)) m1 = 0.f;
  };
  if (NT == 0) finish_first();
  // Where all the tiles this block visits fit the buffers, they are fetched at once and stay for
  // the second visit; else they stream through two buffers (one, where two do not fit), twice.
  const bool resident = NT <= nbuf;
  if (resident) {
    for (int it = 0; it < NT; it++) issue(it, it);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    norms(0, NT);
    __syncthreads();
  } else if (nbuf >= 2) {
    issue(0, 0);
  }
  for (int it = 0; it < total; it++) {
    int buf = 0;
    if (resident) {
      buf = it % NT;
      if (it >= NT) __syncthreads();      // the weights of the tile before have been read
    } else if (nbuf >= 2) {
      buf = it & 1;
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      __syncthreads();
      if (it + 1 < total) issue(it + 1, buf ^ 1);
      norms(buf, 1);
      __syncthreads();
    } else {
      __syncthreads();
      issue(it, 0);
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      __syncthreads();
      norms(0, 1);
      __syncthreads();
    }
    // S: 16 queries x 32 keys of this head
    float s[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
    const uint32_t kb = ks_base + (uint32_t)buf * G * TT_KEYS * DP * 2;
#pragma unroll
    for (int kk = 0; kk < ND16; kk++) {
      uint32_t a[4], al[4], b[4];
      tt_ldsm4(q_addr + kk * 32, a);
      tt_ldsm4(q_addr + q_low + kk * 32, al);
#pragma unroll
      for (int np = 0; np < 2; np++) {
        tt_ldsm4(kb + kb_off + (uint32_t)(np * 16 * DP * 2) + kk * 32, b);
        tt_mma(s[2 * np], al, b[0], b[1]);
        tt_mma(s[2 * np + 1], al, b[2], b[3]);
        tt_mma(s[2 * np], a, b[0], b[1]);
        tt_mma(s[2 * np + 1], a, b[2], b[3]);
      }
    }
    const int key0 = (kt_lo + it % NT) * TT_KEYS;
#pragma unroll
    for (int nt = 0; nt < 4; nt++) {
      const float2 ki = *reinterpret_cast<const float2*>(kinv + (buf * G + c) * TT_KEYS + nt * 8 + c2);
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const int j = key0 + nt * 8 + c2 + (e & 1);
        const int dist = ((e & 2) ? pos1 : pos0) - j;
        const bool vis = ((e & 2) ? ok1 : ok0) && dist >= 0 && (window <= 0 || dist < window);
        s[nt][e] = vis ? s[nt][e] * ((e & 1) ? ki.y : ki.x) * scale2 - slope2 * (float)dist : -INFINITY;
      }
    }
    if (it < NT) {
      // first visit: running maximum and sum of this thread's columns
#pragma unroll
      for (int hf = 0; hf < 2; hf++) {
        float mx = hf ? m1 : m0;
#pragma unroll
        for (int nt = 0; nt < 4; nt++) mx = fmaxf(mx, fmaxf(s[nt][2 * hf], s[nt][2 * hf + 1]));
        if (mx > -INFINITY) {
          float l = (hf ? l1 : l0) * tt_exp2((hf ? m1 : m0) - mx);
#pragma unroll
          for (int nt = 0; nt < 4; nt++) l += tt_exp2(s[nt][2 * hf] - mx) + tt_exp2(s[nt][2 * hf + 1] - mx);
          if (hf) { l1 = l; m1 = mx; } else { l0 = l; m0 = mx; }
        }
      }
      if (it == NT - 1) finish_first();
      continue;
    }
    // second visit: the weights, exchanged, mixed, applied
    float* pw = Ps + (size_t)h * TT_ROWS * TT_PPITCH;
#pragma unroll
    for (int nt = 0; nt < 4; nt++) {
      *reinterpret_cast<float2*>(pw + g4 * TT_PPITCH + nt * 8 + c2) =
          make_float2(tt_exp2(s[nt][0] - m0) * il0, tt_exp2(s[nt][1] - m0) * il0);
      *reinterpret_cast<float2*>(pw + (g4 + 8) * TT_PPITCH + nt * 8 + c2) =
          make_float2(tt_exp2(s[nt][2] - m1) * il1, tt_exp2(s[nt][3] - m1) * il1);
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; i++) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
    for (int g = 0; g < H; g++) {
      const float w = Ts[h * H + g];
      const float* pg = Ps + (size_t)g * TT_ROWS * TT_PPITCH;
#pragma unroll
      for (int nt = 0; nt < 4; nt++) {
        const float2 a = *reinterpret_cast<const float2*>(pg + g4 * TT_PPITCH + nt * 8 + c2);
        const float2 b = *reinterpret_cast<const float2*>(pg + (g4 + 8) * TT_PPITCH + nt * 8 + c2);
        s[nt][0] = fmaf(w, a.x, s[nt][0]);
        s[nt][1] = fmaf(w, a.y, s[nt][1]);
        s[nt][2] = fmaf(w, b.x, s[nt][2]);
        s[nt][3] = fmaf(w, b.y, s[nt][3]);
      }
    }
#pragma unroll
    for (int ks = 0; ks < 2; ks++) {
      uint32_t a[4], b[4];
      a[0] = tt_pack(s[2 * ks][0], s[2 * ks][1]);
      a[1] = tt_pack(s[2 * ks][2], s[2 * ks][3]);
      a[2] = tt_pack(s[2 * ks + 1][0], s[2 * ks + 1][1]);
      a[3] = tt_pack(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
      for (int dp = 0; dp < ND16; dp++) {
        tt_ldsm4_t(kb + vb_off + (uint32_t)(ks * 16 * DP * 2) + dp * 32, b);
        tt_mma(o[2 * dp], a, b[0], b[1]);
        tt_mma(o[2 * dp + 1], a, b[2], b[3]);
      }
    }
  }
  if (S > 1) {
    // the blocks' partial results, added by block 0
#pragma unroll
    for (int hf = 0; hf < 2; hf++) {
      const int row = g4 + 8 * hf;
      if (row >= rows) continue;
#pragma unroll
      for (int nd = 0; nd < 2 * ND16; nd++)
        *reinterpret_cast<float2*>(Os + ((size_t)h * rows + row) * D + nd * 8 + c2) = make_float2(o[nd][2 * hf], o[nd][2 * hf + 1]);
    }
    tt_cluster_sync();
    if (z == 0) {
      for (int zz = 1; zz < S; zz++) {
#pragma unroll
        for (int hf = 0; hf < 2; hf++) {
          const int row = g4 + 8 * hf;
          if (row >= rows) continue;
#pragma unroll
          for (int nd = 0; nd < 2 * ND16; nd++) {
            const float2 v = tt_peer_ld2(tt_peer(Os + ((size_t)h * rows + row) * D + nd * 8 + c2, zz));
            o[nd][2 * hf] += v.x;
            o[nd][2 * hf + 1] += v.y;
          }
        }
      }
    }
    tt_cluster_sync();      // no block leaves while block 0 reads from it
    if (z != 0) return;
  }
  // out = o * mult * sigmoid(gate)
#pragma unroll
  for (int hf = 0; hf < 2; hf++) {
    const int row = g4 + 8 * hf;
    if (row >= rows) continue;
    const size_t t = (size_t)(t0 + row0 + row);
    __nv_bfloat16* op = out + t * o_stride + (size_t)h * D;
    const float* gp = gate ? gate + t * gate_stride + (size_t)h * D : nullptr;
#pragma unroll
    for (int nd = 0; nd < 2 * ND16; nd++) {
      const int d = nd * 8 + c2;
      float x = o[nd][2 * hf] * mult, y = o[nd][2 * hf + 1] * mult;
      if (gp) {
        x *= 1.0f / (1.0f + expf(-gp[d]));
        y *= 1.0f / (1.0f + expf(-gp[d + 1]));
      }
      *reinterpret_cast<__nv_bfloat162*>(op + d) = __floats2bfloat162_rn(x, y);
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

// Tuning hook: 0 keeps one block a tile of queries whatever the grid (default 1: clusters where the
// grid is small).
static int g_tt_split = 1;
SGLC_API void sglc_talk_tiles_set_split(int on) { g_tt_split = on; }

// The tiled form for a bfloat16 cache: requests' new tokens q_start[r] .. q_start[r+1]-1 end at
// position kv_len[r] - 1; max_keys: a bound on kv_len (0: none known).  Head sizes 32, 48, 64, 96 and 128, up to 16 heads, and what fits the
// shared memory of a block; SGLC_ERR_UNSUPPORTED otherwise (the caller then takes the kernel above).
SGLC_API int sglc_talk_attention_tiles(const float* q, long long q_stride, const void* cache, const int* block_table,
                                       int bt_stride, const int* q_start, const int* kv_len, const float* slopes,
                                       const float* talk, const float* gate, long long gate_stride, void* out,
                                       long long o_stride, int R, int max_q_len, int max_keys, int H, int G, int D,
                                       int page_size, float scale, float eps, float mult, int window, int n_pages,
                                       int* err,
                                       cudaStream_t stream) {
  if (R <= 0 || max_q_len <= 0) return SGLC_OK;
  if (H <= 0 || G <= 0 || H % G != 0 || D <= 0 || page_size <= 0 || window < 0) return SGLC_ERR_ARGUMENT;
  if (H > TT_MAX_HEADS || D % 16 != 0 || q_stride % 4 != 0 || o_stride % 2 != 0 || ((uintptr_t)q & 15) != 0 ||
      ((uintptr_t)out & 3) != 0 || ((uintptr_t)cache & 15) != 0)
    return SGLC_ERR_UNSUPPORTED;
  const int rows = max_q_len < TT_ROWS ? max_q_len : TT_ROWS;
  const dim3 tiles((max_q_len + TT_ROWS - 1) / TT_ROWS, R);
  // as many tile buffers as a block's key range can span (window and queries of a tile, or the
  // longest request), if they fit: then every tile is fetched once
  long long span = max_keys > 0 ? max_keys : (1ll << 40);
  if (window > 0 && window + rows - 1 < span) span = window + rows - 1;
  const long long span_tiles = (span + TT_KEYS - 2) / TT_KEYS + 1;
  // few tiles of queries: a cluster of up to 8 blocks shares the key tiles of each
  int split = 1;
  const long long blocks = (long long)tiles.x * tiles.y;
  if (g_tt_split && blocks * 2 <= 128 && span_tiles >= 2) {
    split = (int)(128 / blocks < 8 ? 128 / blocks : 8);
    if (split > span_tiles) split = (int)span_tiles;
  }
  auto smem_for = [&](int nbuf, int S) {
    const size_t DP = D + 8;
    return (size_t)2 * H * TT_ROWS * DP * 2 + (size_t)nbuf * G * TT_KEYS * (DP * 2 + 4) +
           (size_t)H * TT_ROWS * TT_PPITCH * 4 + (size_t)((H * H + 1) & ~1) * 4 +
           (S > 1 ? (size_t)H * TT_ROWS * 2 * 4 + (size_t)H * rows * D * 4 : 0);
  };
  const size_t limit = 227 * 1024;
  if (split > 1 && smem_for(1, split) > limit) split = 1;
  if (smem_for(1, split) > limit) return SGLC_ERR_UNSUPPORTED;
  const long long want = (span_tiles + split - 1) / split;
  int nbuf = 1;
  while (nbuf < want && smem_for(nbuf + 1, split) <= limit) nbuf++;
  if (nbuf < want && nbuf > 2) nbuf = 2;      // streaming uses two
  const size_t smem = smem_for(nbuf, split);
  const dim3 grid(tiles.x, tiles.y, split);
#define TT_GO(ND16)                                                                                              \
  do {                                                                                                           \
    if (smem > 48 * 1024)                                                                                        \
      cudaFuncSetAttribute(talk_tiles_kernel<ND16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
    return sglc_launch(talk_tiles_kernel<ND16>, grid, dim3(H * 32), smem, stream, split, true, q, q_stride,      \
                       (const __nv_bfloat16*)cache, block_table, bt_stride, q_start, kv_len, slopes, talk, gate, \
                       gate_stride, (__nv_bfloat16*)out, o_stride, H, G, page_size, scale, eps, mult, window,    \
                       nbuf, n_pages, err);                                                                      \
  } while (0)
  switch (D) {
    case 32: TT_GO(2);
    case 48: TT_GO(3);
    case 64: TT_GO(4);
    case 96: TT_GO(6);
    case 128: TT_GO(8);
    default: return SGLC_ERR_UNSUPPORTED;
  }
#undef TT_GO
}
