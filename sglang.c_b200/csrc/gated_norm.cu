// The output stage of a recurrent mixer, for the rows of a step: a row of `width` values (one
// head's read-out, or all heads' side by side) is divided by its root mean square,
//   y = o / sqrt(mean(o^2) + eps) * gain * act(gate),
// with a gain of `width` entries that every row of a token shares and a gate of the row's shape
// taken through silu or a sigmoid (or no gate: the norm alone).  Statistics and the gate are 32-bit; the result is written in
// the precision of the product that follows.  A warp a row.
// The general form adds: rows that lie `o_pitch` apart in o (a head's read-out followed by columns
// that are not part of it); a gain of groups x width entries (every row its own); and a divisor per
// row, formed from one more column behind the row and a running maximum m per (token, row):
//   o <- o / (max(|o[width]|, exp(-m)) + 1e-6)      (the read-out of a matrix memory whose state is
//   kept times exp(-m): o[width] is the normaliser's read-out n . q)
// ahead of the norm.
#include "common.cuh"

SGLC_DEFINE_ERROR_STRING()

enum { GN_SILU = 0, GN_SIGMOID = 1, GN_NONE = 2 };   // GN_NONE: no gate at all (gate may be null)

template <typename TO>
__global__ void __launch_bounds__(128)
gated_norm_kernel(const float* __restrict__ o, long long o_stride, const float* __restrict__ gate,
                  long long gate_stride, const float* __restrict__ gain, TO* __restrict__ y, long long y_stride,
                  long long n_rows, int groups, int width, float eps, int act, int o_pitch, int gain_rows,
                  const float* __restrict__ m_run, long long m_stride) {
  pdl_launch_dependents();
  const long long row = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  pdl_wait();
  if (row >= n_rows) return;
  const long long t = row / groups;
  const int c0 = (int)(row % groups) * width;
  const float* op = o + t * o_stride + (row % groups) * o_pitch;
  const float* gp = act == GN_NONE ? nullptr : gate + t * gate_stride + c0;
  if (gain_rows) gain += c0;
  float pre = 1.0f;
  if (m_run) pre = 1.0f / (fmaxf(fabsf(op[width]), expf(-m_run[t * m_stride + row % groups])) + 1e-6f);
  float ss = 0.0f;
  for (int d = lane; d < width; d += 32) {
    const float v = op[d] * pre;
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  const float inv = pre / sqrtf(ss / (float)width + eps);
  TO* yp = y + t * y_stride + c0;
  for (int d = lane; d < width; d += 32) {
    if (act == GN_NONE) {
      yp[d] = from_f32<TO>(op[d] * inv * gain[d]);
      continue;
    }
    const float g = gp[d];
    const float s = 1.0f / (1.0f + expf(-g));
    yp[d] = from_f32<TO>(op[d] * inv * gain[d] * (act == GN_SILU ? g * s : s));
  }
}

// o, gate: float [T][groups*width] (row strides free); gain: float [width]; y: [T][groups*width]
// o_pitch: columns between the rows of a token in o (>= width; width + 1 and more with m_run);
// gain_rows != 0: gain is float [groups*width]; m_run: null, or float [T][groups] (rows m_stride apart).
SGLC_API int sglc_gated_norm_ext(const float* o, long long o_stride, const float* gate, long long gate_stride,
                                 const float* gain, void* y, long long y_stride, int y_dtype, int T, int groups,
                                 int width, float eps, int act, int o_pitch, int gain_rows, const float* m_run,
                                 long long m_stride, cudaStream_t stream) {
  if (T <= 0) return SGLC_OK;
  if (groups <= 0 || width <= 0 || act < GN_SILU || act > GN_NONE || (act != GN_NONE && !gate)) return SGLC_ERR_ARGUMENT;
  if (o_pitch < width + (m_run ? 1 : 0)) return SGLC_ERR_ARGUMENT;
  const long long n_rows = (long long)T * groups;
  const dim3 grid((unsigned)((n_rows + 3) / 4));
  if (y_dtype == SGLC_F32)
    return sglc_launch(gated_norm_kernel<float>, grid, dim3(128), 0, stream, 1, true, o, o_stride, gate, gate_stride,
                       gain, (float*)y, y_stride, n_rows, groups, width, eps, act, o_pitch, gain_rows, m_run, m_stride);
  if (y_dtype == SGLC_BF16)
    return sglc_launch(gated_norm_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, 1, true, o, o_stride, gate,
                       gate_stride, gain, (__nv_bfloat16*)y, y_stride, n_rows, groups, width, eps, act, o_pitch, gain_rows,
                       m_run, m_stride);
  return SGLC_ERR_ARGUMENT;
}

SGLC_API int sglc_gated_norm(const float* o, long long o_stride, const float* gate, long long gate_stride,
                             const float* gain, void* y, long long y_stride, int y_dtype, int T, int groups,
                             int width, float eps, int act, cudaStream_t stream) {
  return sglc_gated_norm_ext(o, o_stride, gate, gate_stride, gain, y, y_stride, y_dtype, T, groups, width, eps, act,
                             width, 0, nullptr, 0, stream);
}
