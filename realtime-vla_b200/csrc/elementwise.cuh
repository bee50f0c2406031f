// Small memory-bound kernels: row normalisations (fp32 residual stream -> bf16 GEMM operand), patch
// extraction, weight repacking and casts.
#pragma once
#include "common.cuh"

enum NormMode { NORM_LAYER = 0, NORM_RMS = 1, NORM_ADARMS = 2 };

// One CTA (128 threads) per row.  x fp32 [rows, D] -> y bf16 [rows, ld_y].
//   NORM_LAYER : (x-mean)*rstd*w + b, eps 1e-5        (w, b fp32 [D])
//   NORM_RMS   : x*rsqrt(mean(x^2)+1e-6)
//   NORM_ADARMS: x*rsqrt(mean(x^2)+1e-6)*(1+style[d]) + style[D+d]     (style fp32 [3*D])
template <int D>
__global__ void __launch_bounds__(128) norm_kernel(const float* __restrict__ x, int ld_x, bf16* __restrict__ y, int ld_y,
                                                   int mode, const float* __restrict__ w, const float* __restrict__ b,
                                                   int in_rpo, int in_obs_stride, int in_row_off) {
  constexpr int PER = (D + 127) / 128;
  __shared__ float red[2][4];
  KTRACE(30);
  pdl_trigger();
  pdl_wait();
  KTRACE(31);
  const int row = blockIdx.x;
  // input row remap: output row r reads input row (r / in_rpo) * in_obs_stride + in_row_off + r % in_rpo
  const int in_row = in_rpo > 0 ? (row / in_rpo) * in_obs_stride + in_row_off + row % in_rpo : row;
  const float* xr = x + (size_t)in_row * ld_x;
  float v[PER];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int d = threadIdx.x + i * 128;
    v[i] = d < D ? xr[d] : 0.f;
    s += (mode == NORM_LAYER) ? v[i] : v[i] * v[i];
  }
  auto block_sum = [&](float val, int slot) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) val += __shfl_xor_sync(0xffffffffu, val, o);
    if ((threadIdx.x & 31) == 0) red[slot][threadIdx.x >> 5] = val;
    __syncthreads();
    return red[slot][0] + red[slot][1] + red[slot][2] + red[slot][3];
  };
  float mean = 0.f, rstd;
  if (mode == NORM_LAYER) {
    mean = block_sum(s, 0) * (1.0f / D);
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int d = threadIdx.x + i * 128;
      const float c = d < D ? v[i] - mean : 0.f;
      q += c * c;
    }
    rstd = rsqrtf(block_sum(q, 1) * (1.0f / D) + 1e-5f);
  } else {
    rstd = rsqrtf(block_sum(s, 0) * (1.0f / D) + 1e-6f);
  }
  bf16* yr = y + (size_t)row * ld_y;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int d = threadIdx.x + i * 128;
    if (d >= D) continue;
    float o;
    if (mode == NORM_LAYER) o = (v[i] - mean) * rstd * w[d] + b[d];
    else if (mode == NORM_RMS) o = v[i] * rstd;
    else o = v[i] * rstd * (1.0f + w[d]) + w[D + d];
    yr[d] = __float2bfloat16(o);
  }
  KTRACE(32);
}

// images bf16 (nv,224,224,3) -> patches bf16 [nv*256, 640]: row = view*256 + py*16 + px, column =
// (iy*14 + ix)*3 + c for the 14x14x3 patch, columns 588..639 zero.
__global__ void patchify_kernel(const bf16* __restrict__ img, bf16* __restrict__ out, int n_rows) {
  pdl_trigger();
  pdl_wait();
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_rows * 640) return;
  const int row = idx / 640, col = idx - row * 640;
  bf16 val = __float2bfloat16(0.f);
  if (col < 588) {
    const int view = row >> 8, py = (row >> 4) & 15, px = row & 15;
    const int iy = col / 42, rem = col - iy * 42;   // rem = ix*3 + c
    val = img[(((size_t)view * 224 + py * 14 + iy) * 224 + px * 14) * 3 + rem];
  }
  out[idx] = val;
}

// W bf16 [K, N] row-major (checkpoint layout) -> Wt bf16 [Np, Kp] row-major, zero padded.
__global__ void repack_kn_to_nk(const bf16* __restrict__ w, int K, int N, bf16* __restrict__ wt, int Kp, int Np) {
  __shared__ bf16 tile[32][33];
  const int n0 = blockIdx.x * 32, k0 = blockIdx.y * 32;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int k = k0 + i, n = n0 + threadIdx.x;
    tile[i][threadIdx.x] = (k < K && n < N) ? w[(size_t)k * N + n] : __float2bfloat16(0.f);
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int n = n0 + i, k = k0 + threadIdx.x;
    if (n < Np && k < Kp) wt[(size_t)n * Kp + k] = tile[threadIdx.x][i];
  }
}

__global__ void bf16_to_f32_kernel(const bf16* __restrict__ in, float* __restrict__ out, size_t n, float scale) {
  pdl_trigger();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = __bfloat162float(in[i]) * scale;
}
__global__ void f32_to_bf16_kernel(const float* __restrict__ in, bf16* __restrict__ out, size_t n) {
  pdl_trigger();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = __float2bfloat16(in[i]);
}
// out[i] = bf16(bf16(in[i]) * scale): a multiply carried out in bf16, as torch does for `w *= s` on a bf16 tensor
__global__ void scale_bf16_kernel(bf16* __restrict__ w, size_t n, float scale) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) w[i] = __float2bfloat16(__bfloat162float(w[i]) * scale);
}
// Start of the action-expert stage: fp32 copy of the bf16 noise, and (Pi0) nothing else.
__global__ void noise_init_kernel(const bf16* __restrict__ noise, float* __restrict__ noise_f32, int n) {
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) noise_f32[i] = __bfloat162float(noise[i]);
}
// prompt embeddings bf16 [L,2048] -> fp32 residual stream rows obs*P + row_off + i, for every observation
__global__ void prompt_rows_kernel(const bf16* __restrict__ emb, float* __restrict__ x, int L, int P, int row_off, int batch) {
  pdl_trigger();
  pdl_wait();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t per = (size_t)L * 2048;
  if (idx >= per * batch) return;
  const int b = (int)(idx / per);
  const size_t r = idx - (size_t)b * per;
  x[((size_t)b * P + row_off) * 2048 + r] = __bfloat162float(emb[r]);
}
// Prompt rows from token ids (pi05_infer.py:769-785: embedding(ids) * sqrt(2048), bf16): row r of the prompt
// window gets bf16(table[ids[r]] * scale) for r < *n_ids and zeros beyond; *n_ids < 0 means the prompt rows
// were given as embeddings and are left alone.  ids and n_ids live in device memory so that the kernel can sit
// inside the captured graph.  An id outside the table is clamped and raises the status word.
__global__ void prompt_from_ids_kernel(const bf16* __restrict__ table, int vocab, const int* __restrict__ ids,
                                       const int* __restrict__ n_ids, bf16* __restrict__ emb, float scale, int* status) {
  pdl_trigger();
  pdl_wait();
  const int n = *n_ids;
  if (n < 0) return;
  const int r = blockIdx.x;
  bf16* dst = emb + (size_t)r * 2048;
  if (r >= n) {
    for (int c = threadIdx.x; c < 2048; c += blockDim.x) dst[c] = __float2bfloat16(0.f);
    return;
  }
  int id = ids[r];
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0 && status) atomicOr(status, VLA_ST_BAD_SHAPE);
    id = min(max(id, 0), vocab - 1);
  }
  const bf16* src = table + (size_t)id * 2048;
  for (int c = threadIdx.x; c < 2048; c += blockDim.x) dst[c] = __float2bfloat16(__bfloat162float(src[c]) * scale);
}
// adaRMS shift rows as a bf16 GEMM operand: style [step][layer][3072] fp32 = [scale | shift | gate] ->
// out [layer][step][1024] bf16 (the shift third), so that shift @ W can be precomputed per (step, layer).
__global__ void style_shift_rows_kernel(const float* __restrict__ style, int n_layers, int n_steps, bf16* __restrict__ out) {
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)n_layers * n_steps * 1024) return;
  const int c = (int)(idx & 1023);
  const int step = (int)((idx >> 10) % n_steps), l = (int)((idx >> 10) / n_steps);
  out[idx] = __float2bfloat16(style[((size_t)step * n_layers + l) * 3072 + 1024 + c]);
}
// dst rows (b*dst_stride + dst_off) <- src rows b, fp32, `width` columns
__global__ void copy_rows_kernel(const float* __restrict__ src, float* __restrict__ dst, int width, int dst_stride_rows,
                                 int dst_off_rows, int batch) {
  pdl_trigger();
  pdl_wait();
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= width * batch) return;
  const int b = idx / width, c = idx - b * width;
  dst[((size_t)b * dst_stride_rows + dst_off_rows) * width + c] = src[(size_t)b * width + c];
}

// Batched forwards: rotary embedding and K/V-cache append as a pass of their own over the bf16 output [tokens, 2560] of
// a plain QKV GEMM (what the reference does with its fused rope/split kernels, pi0_infer.py:777-810).  Inside the GEMM
// this work sits in a per-column epilogue, because 51 suffix rows per observation break every 32-token store block
// across cache rows of two observations; as its own kernel it is one coalesced read and write.
// One block = 32 consecutive tokens (blockIdx.x) x 512 features (blockIdx.y = 0..4).  Token t belongs to observation t / rows_per_obs, local row r = t % rows_per_obs,
// position r + pos_off + *pos_base, cache row obs * kv_obs_stride + kv_row_off + r.  Features [0, 2048) -> q (rotated
// in adjacent pairs), [2048, 2304) -> key cache (rotated), [2304, 2560) -> value cache and, through a transpose in
// shared memory so that the lanes of a store run along the keys, the transposed value cache vt[obs][256][vt_ld].
__global__ void __launch_bounds__(256) qkv_rope_split_kernel(const bf16* __restrict__ qkv, int n_tok, bf16* __restrict__ q,
                                                             bf16* __restrict__ kc, bf16* __restrict__ vc, bf16* __restrict__ vt,
                                                             int vt_ld, const float* __restrict__ rope_cos,
                                                             const float* __restrict__ rope_sin, int pos_off,
                                                             const int* __restrict__ pos_base, int rows_per_obs,
                                                             int kv_obs_stride, int kv_row_off) {
  __shared__ bf16 vtile[32][258];   // [token][dim], rows padded so that the transposed reads hit distinct banks
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int t0 = blockIdx.x * 32;
  const int pb = pos_base ? *pos_base : 0;
  // eight threads per token, 64 consecutive features (eight 16-byte vectors) each: all loads of a thread are issued
  // before the first use, one division per thread
  const int tl = threadIdx.x >> 3, sub = threadIdx.x & 7, t = t0 + tl;
  const int nbase = 512 * blockIdx.y + 64 * sub;
  if (t < n_tok) {
    const int obs = t / rows_per_obs, r = t - obs * rows_per_obs;
    const int pos = r + pos_off + pb;
    const size_t row = (size_t)obs * kv_obs_stride + kv_row_off + r;
    uint4 x[8];
#pragma unroll
    for (int g = 0; g < 8; ++g) x[g] = *reinterpret_cast<const uint4*>(qkv + (size_t)t * 2560 + nbase + 8 * g);
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      const int n = nbase + 8 * g;
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&x[g]);
      if (n < 2304) {
        const int fi = (n & 255) >> 1;
        const float4 c = *reinterpret_cast<const float4*>(rope_cos + pos * 128 + fi);
        const float4 sn = *reinterpret_cast<const float4*>(rope_sin + pos * 128 + fi);
        const float cc[4] = {c.x, c.y, c.z, c.w}, ss[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float v0 = __low2float(h[k]), v1 = __high2float(h[k]);
          h[k] = __floats2bfloat162_rn(v0 * cc[k] - v1 * ss[k], v1 * cc[k] + v0 * ss[k]);
        }
      }
      if (n < 2048) *reinterpret_cast<uint4*>(q + (size_t)t * 2048 + n) = x[g];
      else if (n < 2304) *reinterpret_cast<uint4*>(kc + row * 256 + (n - 2048)) = x[g];
      else {
        *reinterpret_cast<uint4*>(vc + row * 256 + (n - 2304)) = x[g];
#pragma unroll
        for (int k = 0; k < 4; ++k) *reinterpret_cast<__nv_bfloat162*>(&vtile[tl][n - 2304 + 2 * k]) = h[k];
      }
    }
  }
  if (!vt || blockIdx.y != 4) return;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int tk = t0 + lane;
  if (tk < n_tok) {
    const int obs = tk / rows_per_obs, r = tk - obs * rows_per_obs;
    bf16* dst = vt + ((size_t)obs * 256 + warp * 32) * vt_ld + kv_row_off + r;
#pragma unroll 8
    for (int d = 0; d < 32; ++d) dst[(size_t)d * vt_ld] = vtile[lane][warp * 32 + d];
  }
}
