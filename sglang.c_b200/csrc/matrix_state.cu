// Recurrences whose state is a matrix S [D x V] per head and request, in 32-bit floats that
// outlive the step (state[slot][head][D][V]), over the tokens of a step.
//
//   decay form (linear attention with a fixed decay per head):
//       S <- d_h S + k_t v_t^T                         o_t = S^T q_t
//   gated delta rule (per token a decay g_t and a step size b_t, both per head):
//       S <- g_t S;  u = b_t (v_t - S^T k_t);  S <- S + k_t u^T;   o_t = S^T q_t
//   row-gated form (HGRN2: the forget gate of a row also says how much of the value it takes in):
//       f_t = l + (1 - l) sigmoid(x_t)  per head and row, l a learned lower bound in [0, 1);
//       S <- diag(f_t) S + (1 - f_t) v_t^T              o_t = S^T q_t
//     (x_t arrives where the other forms take k_t; the kernel makes f_t as it stages the token)
//   row-decay form (gated linear attention: a decay per key channel and token):
//       a_t = sigmoid(z_t)^(1/tau)  per head and row;   S <- diag(a_t) S + k_t v_t^T;   o_t = S^T q_t
//     (z_t arrives as a third input beside q_t and k_t; the kernel makes a_t as it stages the token)
//   gated form (per token and head a decay g_t and an input weight b_t, made by whoever calls):
//       S <- g_t S + b_t k_t v_t^T                     o_t = S^T q_t
//     with `ones_col` the state has one more column than v has entries, whose "value" is 1 for every
//     token: it carries sum_t b_t k_t under the same decay (a normaliser), and its read-out n_t . q_t
//     leaves in the last column of the head's output.
// in this order: the read-out sees the current token's write.
//
// Column j of S needs nothing of the other columns: S^T k, the update and S^T q are, per column,
// two dot products and one scaled addition over D.  So a column belongs to L lanes of one warp that
// keep it in registers (PER entries each, D <= PER L, entry e of lane s is row PER s + e), a block
// takes a range of columns of one (request, head), and the tokens go by one after the other; the
// block stages the next tokens' q, k, v and gates in shared memory, a batch at a time, while it
// works on the batch before.  A token's time is the time of one warp's chain of dependent
// instructions (measured: 250-290 ns a token at a key size of 64 whether a lane keeps 4, 8 or 16
// entries; 170 ns without the delta rule's first dot product).  PER = 16 costs the fewest
// instructions in all; key sizes of 33..64 take PER = 8 in steps with few (request, head) pairs,
// where it was a tenth faster.
// q and k may have fewer heads than v (head h reads q/k head h / (H / G)).
// With `silu_in` the kernel applies silu to q, k and v as it stages them (row-gated form: to q only).
// `q_scale` multiplies q as it is staged.
#include "common.cuh"

SGLC_DEFINE_ERROR_STRING()

constexpr int MS_UNROLL = 4;      // tokens worked on without a loop between them
constexpr int MS_MAX_DIM = 256;   // key sizes up to 16 entries a lane x 16 lanes

enum { MS_DECAY = 0, MS_DELTA = 1, MS_ROWGATE = 2, MS_ROWDECAY = 3, MS_GATED = 4 };

struct MsArgs {
  const float* q; long long q_stride;     // [T][..], head g at columns g*D
  const float* k; long long k_stride;
  const float* v; long long v_stride;     // head h at columns h*V
  const float* gates; long long gates_stride;   // delta, gated: [T][2H] beta (the input weight) then decay
  const float* row_z; long long row_z_stride;   // row-decay form: [T][G*D] pre-activations of the decays
  float inv_tau;                          // row-decay form: a = exp(log sigmoid(z) * inv_tau)
  float q_scale;                          // a factor of q
  int ones_col;                           // gated form: the state's last column takes the value 1
  const float* head_decay;                // decay form: [H]
  const float* lower;                     // row-gated form: [H*D] lower bounds of the forget gates
  float* out; long long out_stride;       // [T][H*V]
  float* state;                           // [n_slots][H][D][V]
  const int* q_start; const int* state_slots;
  int R, H, G, D, V, n_slots;
  int silu_in;
  int* err;
};

__device__ __forceinline__ float ms_silu(float v) { return v / (1.0f + expf(-v)); }

// L lanes a column, NW warps a block (each warp its own 32 / L columns of one head; the block
// stages q and k once for all of them).  While a batch of tokens is worked on, the next batch's
// loads are in flight into registers; they go to the other half of the staging buffers behind
// the one barrier a batch needs.
template <int MS_PER, int L, int NW, int MODE>
__global__ void __launch_bounds__(32 * NW)
matrix_state_kernel(MsArgs p) {
  // (a lane's entries of q and k lie together in shared memory, 16-byte loads; the stride between
  // lanes is chosen so that the lanes of a quarter warp fall on different banks)
  constexpr int DP = MS_PER * L, THREADS = 32 * NW, COLS = 32 / L * NW, LP = MS_PER == 4 ? 4 : MS_PER + 4, SP = L * LP;
  // Tokens staged at a time: as many as the 48 KB of static shared memory hold, up to 32.  (The loads of a batch are
  // in flight while the batch before is worked on: a batch must take longer than a load's way from
  // memory, about 2 us, or the tokens wait for it; 8 tokens did not.)
  constexpr bool GATES = MODE == MS_DELTA || MODE == MS_GATED, ROWA = MODE == MS_ROWDECAY;
  constexpr int FIT = 6144 / ((ROWA ? 3 : 2) * SP + COLS + 2) / 8 * 8;   // (two halves of q, k, v and gates in 48 KB)
  constexpr int MS_BATCH = FIT >= 32 ? 32 : (FIT >= 8 ? FIT : (ROWA ? 4 : 8));
  constexpr int NG = (2 * MS_BATCH + THREADS - 1) / THREADS;
  constexpr int NK = (MS_BATCH * DP + THREADS - 1) / THREADS;      // q/k entries a thread stages per batch
  constexpr int NV = (MS_BATCH * COLS + THREADS - 1) / THREADS;    // v entries
  __shared__ __align__(16) float ks[2][MS_BATCH * SP], qs[2][MS_BATCH * SP];
  __shared__ float vs[2][MS_BATCH * COLS], gs[2][2 * MS_BATCH];
  __shared__ __align__(16) float as[ROWA ? 2 : 1][ROWA ? MS_BATCH * SP : 4];   // row-decay form: the decays
  pdl_launch_dependents();
  const int r = blockIdx.x, h = blockIdx.y, g = h / (p.H / p.G);
  const int tid = threadIdx.x, sub = tid % L, lcol = tid / L, col = blockIdx.z * COLS + lcol;
  const bool on = col < p.V;
  pdl_wait();
  const int t0 = p.q_start[r], t1 = p.q_start[r + 1];
  const int slot = p.state_slots[r];
  if (t1 <= t0 || !sglc_index_ok(slot, p.n_slots, p.err)) return;
  float* sp = p.state + ((size_t)slot * p.H + h) * p.D * p.V;
  float S[MS_PER];
#pragma unroll
  for (int e = 0; e < MS_PER; e++) {
    const int i = sub * MS_PER + e;
    S[e] = (on && i < p.D) ? sp[(size_t)i * p.V + col] : 0.0f;
  }
  const float hd = MODE == MS_DECAY ? p.head_decay[h] : 0.0f;
  float* out_row = p.out + (size_t)h * p.V + col;
  float rk[NK], rq[NK], rv[NV], rg[NG], ra[ROWA ? NK : 1];
  const int v_in = p.ones_col ? p.V - 1 : p.V;          // entries a head of v has
  auto fetch = [&](int tb) {                 // a batch's inputs into registers (zeros beyond the request's end)
#pragma unroll
    for (int n = 0; n < NK; n++) {
      const int x = tid + n * THREADS, b = x / DP, i = x % DP;
      const bool in = x < MS_BATCH * DP && tb + b < t1 && i < p.D;
      rk[n] = in ? __ldg(p.k + (size_t)(tb + b) * p.k_stride + (size_t)g * p.D + i) : 0.0f;
      rq[n] = in ? __ldg(p.q + (size_t)(tb + b) * p.q_stride + (size_t)g * p.D + i) : 0.0f;
      if (ROWA) ra[n] = in ? __ldg(p.row_z + (size_t)(tb + b) * p.row_z_stride + (size_t)g * p.D + i) : 0.0f;
    }
#pragma unroll
    for (int n = 0; n < NV; n++) {
      const int x = tid + n * THREADS, b = x / COLS, c = blockIdx.z * COLS + x % COLS;
      rv[n] = (x < MS_BATCH * COLS && tb + b < t1 && c < v_in)
                  ? __ldg(p.v + (size_t)(tb + b) * p.v_stride + (size_t)h * v_in + c) : 0.0f;
      if (MODE == MS_GATED && p.ones_col && c == v_in) rv[n] = 1.0f;
    }
    if (GATES) {
      // (beyond the request's end: step size 0, decay 1: such a token leaves the state as it is)
#pragma unroll
      for (int n = 0; n < NG; n++) {
        const int x = tid + n * THREADS, b = x >> 1, which = x & 1;
        rg[n] = (x < 2 * MS_BATCH && tb + b < t1) ? __ldg(p.gates + (size_t)(tb + b) * p.gates_stride + which * p.H + h)
                                                  : (float)which;
      }
    }
  };
  auto stage = [&](int buf) {
#pragma unroll
    for (int n = 0; n < NK; n++) {
      const int x = tid + n * THREADS;
      if (x < MS_BATCH * DP) {
        const int b = x / DP, i = x % DP, at = b * SP + i / MS_PER * LP + i % MS_PER;
        if (MODE == MS_ROWGATE) {
          // What is staged is 1 - f = (1 - l) sigmoid(-x), the share of the value a row takes in:
          // formed from f itself it would lose its digits where f is close to one.
          // (rows beyond the key size take in nothing: their entries stay zero)
          const float lo = i < p.D ? __ldg(p.lower + (size_t)g * p.D + i) : 1.0f;
          ks[buf][at] = (1.0f - lo) * (1.0f / (1.0f + expf(rk[n])));
        } else {
          ks[buf][at] = p.silu_in ? ms_silu(rk[n]) : rk[n];
        }
        qs[buf][at] = (p.silu_in ? ms_silu(rq[n]) : rq[n]) * p.q_scale;
        if (ROWA) {
          // a = sigmoid(z)^(1/tau) = exp(-softplus(-z) / tau)
          const float z = ra[n];
          as[buf][at] = expf(-(fmaxf(-z, 0.0f) + log1pf(expf(-fabsf(z)))) * p.inv_tau);
        }
      }
    }
#pragma unroll
    for (int n = 0; n < NV; n++) {
      const int x = tid + n * THREADS;
      if (x < MS_BATCH * COLS) vs[buf][x] = (p.silu_in && MODE != MS_ROWGATE) ? ms_silu(rv[n]) : rv[n];
    }
    if (GATES) {
#pragma unroll
      for (int n = 0; n < NG; n++)
        if (tid + n * THREADS < 2 * MS_BATCH) gs[buf][tid + n * THREADS] = rg[n];
    }
  };
  fetch(t0);
  int buf = 0;
  for (int tb = t0; tb < t1; tb += MS_BATCH, buf ^= 1) {
    const int nb = min(MS_BATCH, t1 - tb);
    stage(buf);
    __syncthreads();           // the batch is staged; everybody is done with the other half's last batch
    if (tb + MS_BATCH < t1) fetch(tb + MS_BATCH);
    // a token's inputs out of shared memory into registers
    auto take = [&](int b, float (&kk)[MS_PER], float (&qq)[MS_PER], float (&aa)[ROWA ? MS_PER : 1], float& vv,
                    float& beta, float& gd) {
      const float4* kr = reinterpret_cast<const float4*>(ks[buf] + b * SP + sub * LP);
      const float4* qr = reinterpret_cast<const float4*>(qs[buf] + b * SP + sub * LP);
#pragma unroll
      for (int e = 0; e < MS_PER; e += 4) {
        const float4 k4 = kr[e / 4], q4 = qr[e / 4];
        kk[e] = k4.x; kk[e + 1] = k4.y; kk[e + 2] = k4.z; kk[e + 3] = k4.w;
        qq[e] = q4.x; qq[e + 1] = q4.y; qq[e + 2] = q4.z; qq[e + 3] = q4.w;
      }
      if (ROWA) {
        const float4* ar = reinterpret_cast<const float4*>(as[buf] + b * SP + sub * LP);
#pragma unroll
        for (int e = 0; e < MS_PER; e += 4) {
          const float4 a4 = ar[e / 4];
          aa[e] = a4.x; aa[e + 1] = a4.y; aa[e + 2] = a4.z; aa[e + 3] = a4.w;
        }
      }
      vv = vs[buf][b * COLS + lcol];
      if (GATES) { beta = gs[buf][2 * b]; gd = gs[buf][2 * b + 1]; }
      if (MODE == MS_GATED) vv *= beta;
    };
    // the state's update by one token; returns this lane's share of the read-out
    auto update = [&](const float (&kk)[MS_PER], const float (&qq)[MS_PER], const float (&aa)[ROWA ? MS_PER : 1],
                      float vv, float beta, float gd) {
      float o0 = 0.0f, o1 = 0.0f, o2 = 0.0f, o3 = 0.0f;
      if (MODE == MS_DELTA) {
        float d0 = 0.0f, d1 = 0.0f, d2 = 0.0f, d3 = 0.0f;
#pragma unroll
        for (int e = 0; e < MS_PER; e += 4) {
          d0 = fmaf(S[e], kk[e], d0);
          d1 = fmaf(S[e + 1], kk[e + 1], d1);
          d2 = fmaf(S[e + 2], kk[e + 2], d2);
          d3 = fmaf(S[e + 3], kk[e + 3], d3);
        }
        float dk = (d0 + d1) + (d2 + d3);
#pragma unroll
        for (int m = 1; m < L; m <<= 1) dk += __shfl_xor_sync(0xffffffffu, dk, m);
        const float u = beta * (vv - gd * dk);
#pragma unroll
        for (int e = 0; e < MS_PER; e += 4) {
          S[e] = fmaf(kk[e], u, gd * S[e]);
          S[e + 1] = fmaf(kk[e + 1], u, gd * S[e + 1]);
          S[e + 2] = fmaf(kk[e + 2], u, gd * S[e + 2]);
          S[e + 3] = fmaf(kk[e + 3], u, gd * S[e + 3]);
          o0 = fmaf(S[e], qq[e], o0);
          o1 = fmaf(S[e + 1], qq[e + 1], o1);
          o2 = fmaf(S[e + 2], qq[e + 2], o2);
          o3 = fmaf(S[e + 3], qq[e + 3], o3);
        }
      } else if (MODE == MS_ROWGATE) {
#pragma unroll
        for (int e = 0; e < MS_PER; e += 4) {
          S[e] = fmaf(kk[e], vv - S[e], S[e]);
          S[e + 1] = fmaf(kk[e + 1], vv - S[e + 1], S[e + 1]);
          S[e + 2] = fmaf(kk[e + 2], vv - S[e + 2], S[e + 2]);
          S[e + 3] = fmaf(kk[e + 3], vv - S[e + 3], S[e + 3]);
          o0 = fmaf(S[e], qq[e], o0);
          o1 = fmaf(S[e + 1], qq[e + 1], o1);
          o2 = fmaf(S[e + 2], qq[e + 2], o2);
          o3 = fmaf(S[e + 3], qq[e + 3], o3);
        }
      } else if (MODE == MS_ROWDECAY || MODE == MS_GATED) {
        // (gated form: vv arrives times the token's input weight, and every row decays by gd)
        auto dec = [&](int e) {
          if constexpr (ROWA) return aa[e];
          else return gd;
        };
#pragma unroll
        for (int e = 0; e < MS_PER; e += 4) {
          S[e] = fmaf(kk[e], vv, dec(e) * S[e]);
          S[e + 1] = fmaf(kk[e + 1], vv, dec(e + 1) * S[e + 1]);
          S[e + 2] = fmaf(kk[e + 2], vv, dec(e + 2) * S[e + 2]);
          S[e + 3] = fmaf(kk[e + 3], vv, dec(e + 3) * S[e + 3]);
          o0 = fmaf(S[e], qq[e], o0);
          o1 = fmaf(S[e + 1], qq[e + 1], o1);
          o2 = fmaf(S[e + 2], qq[e + 2], o2);
          o3 = fmaf(S[e + 3], qq[e + 3], o3);
        }
      } else {
#pragma unroll
        for (int e = 0; e < MS_PER; e += 4) {
          S[e] = fmaf(kk[e], vv, hd * S[e]);
          S[e + 1] = fmaf(kk[e + 1], vv, hd * S[e + 1]);
          S[e + 2] = fmaf(kk[e + 2], vv, hd * S[e + 2]);
          S[e + 3] = fmaf(kk[e + 3], vv, hd * S[e + 3]);
          o0 = fmaf(S[e], qq[e], o0);
          o1 = fmaf(S[e + 1], qq[e + 1], o1);
          o2 = fmaf(S[e + 2], qq[e + 2], o2);
          o3 = fmaf(S[e + 3], qq[e + 3], o3);
        }
      }
      return (o0 + o1) + (o2 + o3);
    };
    // the read-out summed over the column's lanes and written (a store the compiler knows to be global)
    auto finish = [&](int b, float o) {
#pragma unroll
      for (int m = 1; m < L; m <<= 1) o += __shfl_xor_sync(0xffffffffu, o, m);
      if (on && sub == 0)
        asm volatile("st.global.f32 [%0], %1;" ::"l"(out_row + (size_t)(tb + b) * p.out_stride), "f"(o));
    };
    // Four tokens at a time without a loop between them (eight were a tenth slower: the straight
    // code outgrew what a scheduler keeps of its instructions): a token's inputs leave shared memory
    // while the token before is worked on, and the four read-outs are summed over their lanes together
    // behind the four updates (what is left between two tokens' updates is the chain itself: the
    // dot product, its sum over the lanes, the correction).  The rest of a short batch one by one.
    int b0 = 0;
    for (; b0 + MS_UNROLL <= nb; b0 += MS_UNROLL) {
      float part[MS_UNROLL];
      float kk[2][MS_PER], qq[2][MS_PER], aa[2][ROWA ? MS_PER : 1], vv[2], beta[2] = {0.0f, 0.0f}, gd[2] = {1.0f, 1.0f};
      take(b0, kk[0], qq[0], aa[0], vv[0], beta[0], gd[0]);
#pragma unroll
      for (int b = 0; b < MS_UNROLL; b++) {
        if (b + 1 < MS_UNROLL) take(b0 + b + 1, kk[(b + 1) & 1], qq[(b + 1) & 1], aa[(b + 1) & 1], vv[(b + 1) & 1], beta[(b + 1) & 1], gd[(b + 1) & 1]);
        part[b] = update(kk[b & 1], qq[b & 1], aa[b & 1], vv[b & 1], beta[b & 1], gd[b & 1]);
      }
#pragma unroll
      for (int b = 0; b < MS_UNROLL; b++) finish(b0 + b, part[b]);
    }
    for (; b0 < nb; b0++) {
      float kk[MS_PER], qq[MS_PER], aa[ROWA ? MS_PER : 1], vv, beta = 0.0f, gd = 1.0f;
      take(b0, kk, qq, aa, vv, beta, gd);
      finish(b0, update(kk, qq, aa, vv, beta, gd));
    }
  }
#pragma unroll
  for (int e = 0; e < MS_PER; e++) {
    const int i = sub * MS_PER + e;
    if (on && i < p.D) sp[(size_t)i * p.V + col] = S[e];
  }
}

template <int PER, int MODE, int NW>
static int ms_launch(const MsArgs& p, int L, dim3 grid, cudaStream_t stream) {
#define MS_CASE(LL)                                                                                         \
  case LL:                                                                                                  \
    if constexpr (PER == 16 ? PER * LL <= MS_MAX_DIM : PER * LL == 64)                                \
      return sglc_launch(matrix_state_kernel<PER, LL, NW, MODE>, grid, dim3(32 * NW), 0, stream, 1, true, p); \
    break;
  switch (L) {
    MS_CASE(1) MS_CASE(2) MS_CASE(4) MS_CASE(8) MS_CASE(16) MS_CASE(32)
  }
#undef MS_CASE
  return SGLC_ERR_UNSUPPORTED;
}

// Tuning hook: 0 (default) lets the launcher choose the entries a lane keeps; 8 or 16 fixes them where legal.
static int g_ms_per = 0;
SGLC_API void sglc_matrix_state_set_per(int per) { g_ms_per = per; }

// mode 0: decay form (head_decay [H]); mode 1: gated delta rule (gates [T][2H]: beta, decay).
// q, k: float rows with G heads of D; v: H heads of V; out: [T][H*V] float; state [n_slots][H][D][V].
// mode 2: row-gated form (k holds the gates' pre-activations, lower [H*D] their lower bounds; G == H).
// mode 3: row-decay form (row_z [T][G*D] the decays' pre-activations, inv_tau = 1 / tau).
// mode 4: gated form (gates [T][2H]: input weight, decay); ones_col: the state has V columns of which
// the last takes the value 1 (v then has heads of V - 1 entries; out still has heads of V).
// q_scale: a factor of q (1 for none).
SGLC_API int sglc_matrix_state_gen(int mode, const float* q, long long q_stride, const float* k, long long k_stride,
                                   const float* v, long long v_stride, const float* gates, long long gates_stride,
                                   const float* head_decay, const float* lower, const float* row_z,
                                   long long row_z_stride, float inv_tau, float q_scale, int ones_col, float* out,
                                   long long out_stride, float* state, int n_slots, const int* q_start,
                                   const int* state_slots, int R, int H, int G, int D, int V, int silu_in, int* err,
                                   cudaStream_t stream) {
  if (R <= 0) return SGLC_OK;
  if (H <= 0 || G <= 0 || H % G != 0 || D <= 0 || V <= 0) return SGLC_ERR_ARGUMENT;
  if (D > MS_MAX_DIM || H > 65535) return SGLC_ERR_UNSUPPORTED;
  MsArgs p = {};
  p.q = q; p.q_stride = q_stride; p.k = k; p.k_stride = k_stride; p.v = v; p.v_stride = v_stride;
  p.gates = gates; p.gates_stride = gates_stride; p.head_decay = head_decay; p.lower = lower;
  p.out = out; p.out_stride = out_stride; p.state = state; p.q_start = q_start; p.state_slots = state_slots;
  p.R = R; p.H = H; p.G = G; p.D = D; p.V = V; p.n_slots = n_slots; p.silu_in = silu_in; p.err = err;
  p.row_z = row_z; p.row_z_stride = row_z_stride; p.inv_tau = inv_tau; p.q_scale = q_scale;
  p.ones_col = mode == MS_GATED && ones_col ? 1 : 0;
  if (p.ones_col && V < 2) return SGLC_ERR_ARGUMENT;
  // Entries a lane keeps: 8 for key sizes of 33..64 while the warps still find a scheduler each (two
  // on each of the 148 x 4); else 16.
  auto lanes = [&](int per) { int l = 1; while (per * l < D) l <<= 1; return l; };
  auto warps = [&](int per) { const int wc = 32 / lanes(per); return (long long)R * H * ((V + wc - 1) / wc); };
  int per = 16;
  for (int cand : {8}) {
    const bool legal = cand * lanes(cand) == 64;      // (the kernels that exist)
    if (legal && (g_ms_per == cand || (g_ms_per == 0 && warps(cand) <= 148LL * 4 * 2))) { per = cand; break; }
  }
  const int L = lanes(per);
  // a warp takes 32 / L columns; four warps a block where a head has columns for more than one
  const int wcols = 32 / L;
  const int NW = V > wcols ? 4 : 1;
  const int zb = (V + wcols * NW - 1) / (wcols * NW);
  if (zb > 65535) return SGLC_ERR_UNSUPPORTED;
  const dim3 grid(R, H, zb);
#define MS_GO(MODE)                                                                                   \
  do {                                                                                                \
    if (per == 8) return NW == 4 ? ms_launch<8, MODE, 4>(p, L, grid, stream) : ms_launch<8, MODE, 1>(p, L, grid, stream);   \
    return NW == 4 ? ms_launch<16, MODE, 4>(p, L, grid, stream) : ms_launch<16, MODE, 1>(p, L, grid, stream);               \
  } while (0)
  if (mode == MS_DECAY) {
    if (!head_decay) return SGLC_ERR_ARGUMENT;
    MS_GO(MS_DECAY);
  }
  if (mode == MS_DELTA) {
    if (!gates) return SGLC_ERR_ARGUMENT;
    MS_GO(MS_DELTA);
  }
  if (mode == MS_ROWGATE) {
    if (!lower || G != H) return SGLC_ERR_ARGUMENT;
    MS_GO(MS_ROWGATE);
  }
  if (mode == MS_ROWDECAY) {
    if (!row_z) return SGLC_ERR_ARGUMENT;
    MS_GO(MS_ROWDECAY);
  }
  if (mode == MS_GATED) {
    if (!gates) return SGLC_ERR_ARGUMENT;
    MS_GO(MS_GATED);
  }
  return SGLC_ERR_ARGUMENT;
}

SGLC_API int sglc_matrix_state_ext(int mode, const float* q, long long q_stride, const float* k, long long k_stride,
                                   const float* v, long long v_stride, const float* gates, long long gates_stride,
                                   const float* head_decay, const float* lower, float* out, long long out_stride,
                                   float* state, int n_slots, const int* q_start, const int* state_slots, int R, int H,
                                   int G, int D, int V, int silu_in, int* err, cudaStream_t stream) {
  if (mode > MS_ROWGATE) return SGLC_ERR_ARGUMENT;
  return sglc_matrix_state_gen(mode, q, q_stride, k, k_stride, v, v_stride, gates, gates_stride, head_decay, lower,
                               nullptr, 0, 0.0f, 1.0f, 0, out, out_stride, state, n_slots, q_start, state_slots, R, H, G,
                               D, V, silu_in, err, stream);
}

SGLC_API int sglc_matrix_state(int mode, const float* q, long long q_stride, const float* k, long long k_stride,
                               const float* v, long long v_stride, const float* gates, long long gates_stride,
                               const float* head_decay, float* out, long long out_stride, float* state,
                               int n_slots, const int* q_start, const int* state_slots, int R, int H, int G,
                               int D, int V, int silu_in, int* err, cudaStream_t stream) {
  if (mode == MS_ROWGATE) return SGLC_ERR_ARGUMENT;
  return sglc_matrix_state_ext(mode, q, q_stride, k, k_stride, v, v_stride, gates, gates_stride, head_decay, nullptr, out,
                               out_stride, state, n_slots, q_start, state_slots, R, H, G, D, V, silu_in, err, stream);
}

// Exponential gates with a running maximum (the gates of a matrix memory with exponential input
// gate, mLSTM): per token and head, from the pre-activations x_i, x_f,
//   i = cap tanh(x_i / cap),   f = log sigmoid(cap tanh(x_f / cap)),
//   m_t = max(f + m_(t-1), i)          (m starts at 0 for a new request and is carried per request)
//   decay_t = exp(f + m_(t-1) - m_t),  weight_t = exp(i - m_t)
// so that a state kept as S_t = decay_t S_(t-1) + weight_t (...) is the true state times exp(-m_t).
// Results: gates [T][2H] (weight, then decay: what the gated form of the recurrence above takes) and
// m_t [T][H].  A warp a (request, head): 32 tokens at a time, a lane a token; the recurrence of m is
// a scan under (f, i) o (f', i') = (f + f', max(i + f', i')), done by shuffles.  Whatever rounding
// the order of that scan leaves in m_t cancels: decay, weight and whoever reads m_t use the same m_t.
__global__ void __launch_bounds__(128)
stabilized_gates_kernel(const float* __restrict__ xi, long long xi_stride, const float* __restrict__ xf,
                        long long xf_stride, float cap, float* __restrict__ gates, long long gates_stride,
                        float* __restrict__ m_out, long long m_stride, float* __restrict__ m_state, int n_slots,
                        const int* __restrict__ q_start, const int* __restrict__ state_slots, int R, int H, int* err) {
  pdl_launch_dependents();
  const int r = blockIdx.x, h = blockIdx.y * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  pdl_wait();
  if (h >= H) return;
  const int t0 = q_start[r], t1 = q_start[r + 1];
  const int slot = state_slots[r];
  if (t1 <= t0 || !sglc_index_ok(slot, n_slots, err)) return;
  float m_in = m_state[(size_t)slot * H + h];
  const float inv_cap = 1.0f / cap;
  // (the next 32 tokens' pre-activations are asked for before these tokens' arithmetic: a batch
  // then costs its chain of shuffles and exponentials, not a trip to memory on top)
  float zi_next = 0.0f, zf_next = 0.0f;
  if (t0 + lane < t1) {
    zi_next = xi[(size_t)(t0 + lane) * xi_stride + h];
    zf_next = xf[(size_t)(t0 + lane) * xf_stride + h];
  }
  for (int tb = t0; tb < t1; tb += 32) {
    const int t = tb + lane;
    const bool on = t < t1;
    float f = 0.0f, i = -INFINITY;            // beyond the end: the identity of the scan
    const float zi = zi_next, zf = zf_next;
    if (t + 32 < t1) {
      zi_next = xi[(size_t)(t + 32) * xi_stride + h];
      zf_next = xf[(size_t)(t + 32) * xf_stride + h];
    }
    if (on) {
      i = cap * tanhf(zi * inv_cap);
      const float u = cap * tanhf(zf * inv_cap);
      f = -(fmaxf(-u, 0.0f) + log1pf(expf(-fabsf(u))));
    }
    float a = f, b = i;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float ap = __shfl_up_sync(0xffffffffu, a, o), bp = __shfl_up_sync(0xffffffffu, b, o);
      if (lane >= o) {
        b = fmaxf(bp + a, b);
        a = ap + a;
      }
    }
    const float m = fmaxf(a + m_in, b);
    float mp = __shfl_up_sync(0xffffffffu, m, 1);
    if (lane == 0) mp = m_in;
    if (on) {
      gates[(size_t)t * gates_stride + h] = expf(i - m);
      gates[(size_t)t * gates_stride + H + h] = expf(f + mp - m);
      m_out[(size_t)t * m_stride + h] = m;
    }
    m_in = __shfl_sync(0xffffffffu, m, 31);
  }
  if (lane == 0) m_state[(size_t)slot * H + h] = m_in;
}

// xi, xf: float [T][..] with the heads' pre-activations at columns 0..H-1 of each pointer; gates: float
// [T][2H]; m_out: float [T][H]; m_state: float [n_slots][H], read and written for the requests' slots.
SGLC_API int sglc_stabilized_gates(const float* xi, long long xi_stride, const float* xf, long long xf_stride, float cap,
                                   float* gates, long long gates_stride, float* m_out, long long m_stride,
                                   float* m_state, int n_slots, const int* q_start, const int* state_slots, int R,
                                   int H, int* err, cudaStream_t stream) {
  if (R <= 0) return SGLC_OK;
  if (H <= 0 || !(cap > 0.0f)) return SGLC_ERR_ARGUMENT;
  if ((H + 3) / 4 > 65535) return SGLC_ERR_UNSUPPORTED;
  return sglc_launch(stabilized_gates_kernel, dim3(R, (H + 3) / 4), dim3(128), 0, stream, 1, true, xi, xi_stride, xf,
                     xf_stride, cap, gates, gates_stride, m_out, m_stride, m_state, n_slots, q_start, state_slots, R, H,
                     err);
}
