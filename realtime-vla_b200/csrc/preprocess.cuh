// Kernels either side of the forward in a robot loop (the reference does these on the host with PIL / numpy in
// its evaluation script, test.py:82-151, 180-204): camera frame -> normalised model input, robot state -> model
// input, action chunk -> robot command.  All of it is small, byte/integer or float64 work bound by memory
// latency, written so that the results are bit-identical to the host code.
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

constexpr int PP_PRECISION_BITS = 32 - 8 - 2;   // Pillow's 8-bit resample keeps coefficients in 22-bit fixed point

__device__ __forceinline__ uint8_t pp_clip8(int acc) {
  const int v = acc >> PP_PRECISION_BITS;       // arithmetic shift, as in the C source
  return (uint8_t)min(max(v, 0), 255);
}

// Horizontal pass of the bilinear resample: in uint8 [H][W][3] -> tmp uint8 [H][rw][3].
// bounds[2*xx] = first input column, bounds[2*xx+1] = tap count, kk[xx*ksize + t] = fixed-point weight.
__global__ void pp_resize_h_kernel(const uint8_t* __restrict__ in, int H, int W, uint8_t* __restrict__ tmp, int rw,
                                   const int* __restrict__ bounds, const int* __restrict__ kk, int ksize) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= H * rw) return;
  const int y = idx / rw, xx = idx - y * rw;
  const int x0 = bounds[2 * xx], n = bounds[2 * xx + 1];
  const int* k = kk + (size_t)xx * ksize;
  const uint8_t* p = in + ((size_t)y * W + x0) * 3;
  int a0 = 1 << (PP_PRECISION_BITS - 1), a1 = a0, a2 = a0;
  for (int t = 0; t < n; ++t) {
    const int w = k[t];
    a0 += p[3 * t] * w;
    a1 += p[3 * t + 1] * w;
    a2 += p[3 * t + 2] * w;
  }
  uint8_t* o = tmp + (size_t)idx * 3;
  o[0] = pp_clip8(a0);
  o[1] = pp_clip8(a1);
  o[2] = pp_clip8(a2);
}

// Vertical pass + paste on the black 224x224 canvas + x/255*2-1 (float32, no contraction) + bf16.
// tmp uint8 [H][rw][3] -> out bf16 [224][224][3]; the resized picture is rh x rw at (pad_h, pad_w).
__global__ void pp_resize_v_pad_norm_kernel(const uint8_t* __restrict__ tmp, int H, int rw, int rh, int pad_h, int pad_w,
                                            const int* __restrict__ bounds, const int* __restrict__ kk, int ksize,
                                            __nv_bfloat16* __restrict__ out) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= 224 * 224) return;
  const int oy = idx / 224, ox = idx - oy * 224;
  const int yy = oy - pad_h, x = ox - pad_w;
  int v0 = 0, v1 = 0, v2 = 0;
  if (yy >= 0 && yy < rh && x >= 0 && x < rw) {
    const int y0 = bounds[2 * yy], n = bounds[2 * yy + 1];
    const int* k = kk + (size_t)yy * ksize;
    int a0 = 1 << (PP_PRECISION_BITS - 1), a1 = a0, a2 = a0;
    for (int t = 0; t < n; ++t) {
      const uint8_t* p = tmp + ((size_t)(y0 + t) * rw + x) * 3;
      const int w = k[t];
      a0 += p[0] * w;
      a1 += p[1] * w;
      a2 += p[2] * w;
    }
    v0 = pp_clip8(a0);
    v1 = pp_clip8(a1);
    v2 = pp_clip8(a2);
  }
  __nv_bfloat16* o = out + (size_t)idx * 3;
  o[0] = __float2bfloat16_rn(__fsub_rn(__fmul_rn(__fdiv_rn((float)v0, 255.0f), 2.0f), 1.0f));
  o[1] = __float2bfloat16_rn(__fsub_rn(__fmul_rn(__fdiv_rn((float)v1, 255.0f), 2.0f), 1.0f));
  o[2] = __float2bfloat16_rn(__fsub_rn(__fmul_rn(__fdiv_rn((float)v2, 255.0f), 2.0f), 1.0f));
}

// State normalisation in float64 without contraction, then float32, then bf16, zero-padded to 32.
// mode 0: (s - mean) / (std + 1e-6); mode 1: (s - q01) / (q99 - q01 + 1e-6) * 2 - 1.  vec = [state n][a n][b n].
__global__ void pp_state_kernel(const double* __restrict__ vec, int n, int mode, __nv_bfloat16* __restrict__ out,
                                double* __restrict__ out_f64) {
  const int i = threadIdx.x;
  if (i >= 32) return;
  double v = 0.0;
  if (i < n) {
    const double s = vec[i], a = vec[n + i], b = vec[2 * n + i];
    if (mode == 0) v = __ddiv_rn(__dsub_rn(s, a), __dadd_rn(b, 1e-6));
    else v = __dsub_rn(__dmul_rn(__ddiv_rn(__dsub_rn(s, a), __dadd_rn(__dsub_rn(b, a), 1e-6)), 2.0), 1.0);
  }
  if (out) out[i] = __float2bfloat16_rn((float)v);
  if (out_f64) out_f64[i] = v;
}

// Action chunk -> robot command, float64: un-normalise (mode 0: a*(std+1e-6)+mean; mode 1:
// (a+1)/2*(q99-q01+1e-6)+q01; statistics beyond n_stats are zero), keep the first action_dim columns, add the raw
// state (delta -> absolute); the last dimension of every 7-wide arm gets the state subtracted again.
// vec = [a n_stats][b n_stats][state n_state].
__global__ void pp_actions_kernel(const __nv_bfloat16* __restrict__ actions, int chunk, const double* __restrict__ vec,
                                  int n_stats, int n_state, int mode, int action_dim, double* __restrict__ out) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= chunk * action_dim) return;
  const int r = idx / action_dim, j = idx - r * action_dim;
  const double act = (double)__bfloat162float(actions[r * 32 + j]);
  const double a = j < n_stats ? vec[j] : 0.0, b = j < n_stats ? vec[n_stats + j] : 0.0;
  double v;
  if (mode == 0) v = __dadd_rn(__dmul_rn(act, __dadd_rn(b, 1e-6)), a);
  else v = __dadd_rn(__dmul_rn(__ddiv_rn(__dadd_rn(act, 1.0), 2.0), __dadd_rn(__dsub_rn(b, a), 1e-6)), a);
  const double s = j < n_state ? vec[2 * n_stats + j] : 0.0;
  v = __dadd_rn(v, s);
  if ((j % 7) == 6 && j < (action_dim / 7) * 7) v = __dsub_rn(v, s);
  out[idx] = v;
}
