// Routing of a mixture of experts for the tokens of a step, from 32-bit router logits z [T][E]:
//   s = sigmoid(z);   choice = s + correction          (the correction only steers the choice)
//   experts form `n_groups` equal groups of neighbours; a group's score is the sum of its two
//   largest choice scores; only experts of the `keep` best groups can be chosen (the others
//   count as minus infinity); the `top` largest choice scores among them are chosen;
//   a chosen expert's weight is its s (times `weight_scale`; with `renorm` the chosen weights
//   are first divided by their sum plus `renorm_eps`).
// `score_fn` 1: s = softmax(z) over all experts instead of the sigmoid.
// Ties go to the lower index.  Results: dense [T][E] weights (zero where not chosen), and the
// chosen ids and weights [T][top] in order of choice.  A thread a token; all 32-bit.
#include "common.cuh"

SGLC_DEFINE_ERROR_STRING()

constexpr int ROUTER_MAX_EXPERTS = 256;
constexpr int ROUTER_MAX_GROUPS = 64;

__global__ void __launch_bounds__(64)
router_kernel(const float* __restrict__ z, long long z_stride, const float* __restrict__ correction,
              float* __restrict__ dense, long long dense_stride, int* __restrict__ ids, float* __restrict__ wts,
              int T, int E, int top, int n_groups, int keep, int renorm, float weight_scale, int score_fn,
              float renorm_eps) {
  pdl_launch_dependents();
  const int t = blockIdx.x * 64 + threadIdx.x;
  pdl_wait();
  if (t >= T) return;
  float c[ROUTER_MAX_EXPERTS];
  float gscore[ROUTER_MAX_GROUPS];
  const float* zr = z + (size_t)t * z_stride;
  float zmax = -INFINITY, zden = 1.0f;
  if (score_fn == 1) {                         // softmax: the largest logit and the sum of exponentials
    for (int e = 0; e < E; e++) zmax = fmaxf(zmax, zr[e]);
    zden = 0.0f;
    for (int e = 0; e < E; e++) zden += expf(zr[e] - zmax);
  }
  for (int e = 0; e < E; e++) {
    const float s = score_fn == 1 ? expf(zr[e] - zmax) / zden : 1.0f / (1.0f + expf(-zr[e]));
    c[e] = s + (correction ? correction[e] : 0.0f);
    dense[(size_t)t * dense_stride + e] = 0.0f;
  }
  if (n_groups > 1 && keep < n_groups) {
    const int per = E / n_groups;
    for (int g = 0; g < n_groups; g++) {
      float a = -INFINITY, b = -INFINITY;      // largest, second largest
      for (int e = g * per; e < (g + 1) * per; e++) {
        const float v = c[e];
        if (v > a) { b = a; a = v; }
        else if (v > b) b = v;
      }
      gscore[g] = per > 1 ? a + b : a;
    }
    // the groups that stay: the `keep` best; the others' experts leave the choice
    unsigned long long kept = 0ull;
    for (int n = 0; n < keep; n++) {
      int best = -1;
      for (int g = 0; g < n_groups; g++)
        if (!((kept >> g) & 1ull) && (best < 0 || gscore[g] > gscore[best])) best = g;
      kept |= 1ull << best;
    }
    for (int g = 0; g < n_groups; g++)
      if (!((kept >> g) & 1ull))
        for (int e = g * per; e < (g + 1) * per; e++) c[e] = -INFINITY;
  }
  float sum = 0.0f;
  for (int n = 0; n < top; n++) {
    int best = -1;
    for (int e = 0; e < E; e++)
      if (!isnan(c[e]) && (best < 0 || c[e] > c[best])) best = e;
    const float s = score_fn == 1 ? expf(zr[best] - zmax) / zden : 1.0f / (1.0f + expf(-zr[best]));
    ids[(size_t)t * top + n] = best;
    wts[(size_t)t * top + n] = s;
    sum += s;
    c[best] = NAN;                             // taken
  }
  const float f = (renorm ? 1.0f / (sum + renorm_eps) : 1.0f) * weight_scale;
  for (int n = 0; n < top; n++) {
    const float w = wts[(size_t)t * top + n] * f;
    wts[(size_t)t * top + n] = w;
    dense[(size_t)t * dense_stride + ids[(size_t)t * top + n]] = w;
  }
}

SGLC_API int sglc_router_ext(const float* z, long long z_stride, const float* correction, float* dense,
                             long long dense_stride, int* ids, float* wts, int T, int E, int top, int n_groups,
                             int keep, int renorm, float weight_scale, int score_fn, float renorm_eps,
                             cudaStream_t stream) {
  if (T <= 0) return SGLC_OK;
  if (E <= 0 || top <= 0 || top > E || n_groups < 1 || E % n_groups != 0 || keep < 1 || keep > n_groups)
    return SGLC_ERR_ARGUMENT;
  if (E > ROUTER_MAX_EXPERTS || n_groups > ROUTER_MAX_GROUPS) return SGLC_ERR_UNSUPPORTED;
  if (n_groups > 1 && keep < n_groups && top > keep * (E / n_groups)) return SGLC_ERR_ARGUMENT;
  if (score_fn != 0 && score_fn != 1) return SGLC_ERR_ARGUMENT;
  return sglc_launch(router_kernel, dim3((T + 63) / 64), dim3(64), 0, stream, 1, true, z, z_stride, correction, dense,
                     dense_stride, ids, wts, T, E, top, n_groups, keep, renorm, weight_scale, score_fn, renorm_eps);
}

SGLC_API int sglc_router(const float* z, long long z_stride, const float* correction, float* dense,
                         long long dense_stride, int* ids, float* wts, int T, int E, int top, int n_groups,
                         int keep, int renorm, float weight_scale, cudaStream_t stream) {
  return sglc_router_ext(z, z_stride, correction, dense, dense_stride, ids, wts, T, E, top, n_groups, keep, renorm,
                         weight_scale, 0, 0.0f, stream);
}
