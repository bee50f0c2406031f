// Softmax attention for the three attention shapes of the path (ViT 16 heads x 72, prefix MQA and
// suffix MQA with head dim 256).  Queries are plain rows: with one shared K/V head, the 8 query heads of
// a token are 8 consecutive query rows (row = token*8 + head).
//
// One CTA = 64 query rows (4 warps x 16 rows), streaming 64-key blocks through shared memory, online
// softmax, bf16 mma.sync (m16n8k16) with fp32 accumulation.  The keys can be split over the CTAs of a
// cluster (grid.x = cluster size); the partial (max, sum, output) triples are merged in fixed order through
// a small global scratch that stays in L2 (distributed shared memory was several times slower for this
// all-to-all pattern).  No logits or probabilities are written to global memory.
//
// Visibility of key j for query row i:
//     j < n_keys  &&  ( j < valid_prefix  ||  ( j >= prefix_alloc && (i >= restrict_rows || j <= prefix_alloc) ) )
// which covers: no mask (valid_prefix = prefix_alloc = n_keys), the Pi05 prefix-length mask, the Pi0
// state-token rule (its 8 head rows see the prefix and suffix key 0 only) and the Pi05 suffix mask.
#pragma once
#include "common.cuh"

struct AttnParams {
  const bf16* q; const bf16* k; const bf16* v; bf16* o;
  int ldq, ldk, ldv, ldo;                 // row strides in elements
  long long q_go, q_gi, k_go, k_gi, v_go, v_gi, o_go, o_gi;   // group offsets: outer (observation/view), inner (head)
  int g_inner;                            // groups = outer * inner, blockIdx.z = outer * g_inner + inner
  int n_q, n_keys;
  int prefix_alloc;
  int valid_prefix;                       // used when valid_prefix_ptr is null
  const int* valid_prefix_ptr;            // optional device scalar
  int restrict_rows;
  float scale_log2e;                      // softmax scale * log2(e)
  int ksplit;                             // cluster size along keys
  float* scratch;                         // partial outputs of the key splits (ksplit > 1)
};

__device__ __forceinline__ void ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;   // size 0 -> the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

template <int HD>
struct AttnCfg {
  static constexpr int HDP = (HD + 15) / 16 * 16;        // head dim padded to the MMA K step
  static constexpr int ROW_BYTES = HDP * 2 + 16;         // +16 B keeps ldmatrix rows on distinct banks
  static constexpr int CHUNKS = HD * 2 / 16;             // 16-byte chunks of real data per row
  static constexpr int TILE_BYTES = 64 * ROW_BYTES;
  static constexpr int KV_BUFS = 2;
  static constexpr int KV_BYTES = 2 * KV_BUFS * TILE_BYTES;
  static constexpr int SMEM_BYTES = TILE_BYTES + KV_BYTES + 16;
  static constexpr int SCRATCH_ROW_FLOATS = HDP + 4;     // per query row and key split: outputs, max, sum
};

// Load a 64-row tile (rows row0.. of a [*, ld] matrix, HD real columns) into padded shared memory.
template <int HD>
__device__ __forceinline__ void attn_load_tile(uint32_t dst, const bf16* src, int ld, int row0, int n_rows) {
  using C = AttnCfg<HD>;
  for (int i = threadIdx.x; i < 64 * C::CHUNKS; i += 128) {
    const int r = i / C::CHUNKS, c = i - r * C::CHUNKS;
    const bool ok = row0 + r < n_rows;
    const bf16* s = src + (size_t)(ok ? row0 + r : 0) * ld + c * 8;
    cp_async16(dst + r * C::ROW_BYTES + c * 16, s, ok);
  }
}

template <int HD>
__global__ void __launch_bounds__(128, 1) attention_kernel(const AttnParams p) {
  using C = AttnCfg<HD>;
  constexpr int KSTEPS = C::HDP / 16;      // MMA k-steps over the head dim (QK^T)
  constexpr int DT = C::HDP / 8;           // 8-wide output tiles over the head dim (PV)
  extern __shared__ __align__(16) uint8_t smem[];
  const uint32_t sQ = smem_u32(smem);
  const uint32_t sKV = sQ + C::TILE_BYTES;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tq = lane & 3;
  const int rank = blockIdx.x, ksplit = p.ksplit;
  const int row0 = blockIdx.y * 64;
  const int go = blockIdx.z / p.g_inner, gi = blockIdx.z - go * p.g_inner;
  const bf16* Q = p.q + go * p.q_go + gi * p.q_gi;
  const bf16* K = p.k + go * p.k_go + gi * p.k_gi;
  const bf16* V = p.v + go * p.v_go + gi * p.v_gi;
  bf16* O = p.o + go * p.o_go + gi * p.o_gi;

  // zero the pad columns once (only HD=72 has any): Q/K pads feed the QK^T k-loop, V pads feed unused outputs
  if (C::HDP != HD) {
    for (int i = threadIdx.x; i < 64 * (1 + 2 * C::KV_BUFS); i += 128) {
      uint8_t* rowp = smem + i * C::ROW_BYTES + HD * 2;
      for (int b = 0; b < (C::HDP - HD) * 2; b += 4) *reinterpret_cast<uint32_t*>(rowp + b) = 0u;
    }
  }
  KTRACE(20);
  pdl_trigger();
  pdl_wait();
  KTRACE(21);

  const int valid_prefix = p.valid_prefix_ptr ? min(max(*p.valid_prefix_ptr, 0), p.prefix_alloc) : p.valid_prefix;

  // keys handled by this CTA: 64-key blocks [blk_begin, blk_end)
  const int n_blk = (p.n_keys + 63) / 64;
  const int blk_begin = (int)(((long long)rank * n_blk) / ksplit);
  const int blk_end = (int)(((long long)(rank + 1) * n_blk) / ksplit);

  attn_load_tile<HD>(sQ, Q, p.ldq, row0, p.n_q);
  if (blk_begin < blk_end) {
    attn_load_tile<HD>(sKV, K, p.ldk, blk_begin * 64, p.n_keys);
    attn_load_tile<HD>(sKV + C::KV_BUFS * C::TILE_BYTES, V, p.ldv, blk_begin * 64, p.n_keys);
  }
  cp_async_commit();

  float acc[DT][4];
#pragma unroll
  for (int i = 0; i < DT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
  float m_run[2] = {-1e30f, -1e30f}, l_run[2] = {0.f, 0.f};
  const int qrow[2] = {row0 + warp * 16 + g, row0 + warp * 16 + g + 8};

  for (int blk = blk_begin; blk < blk_end; ++blk) {
    const int buf = (blk - blk_begin) & 1;
    if (blk + 1 < blk_end) {
      attn_load_tile<HD>(sKV + (buf ^ 1) * C::TILE_BYTES, K, p.ldk, (blk + 1) * 64, p.n_keys);
      attn_load_tile<HD>(sKV + (C::KV_BUFS + (buf ^ 1)) * C::TILE_BYTES, V, p.ldv, (blk + 1) * 64, p.n_keys);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const uint32_t sK = sKV + buf * C::TILE_BYTES;
    const uint32_t sV = sKV + (C::KV_BUFS + buf) * C::TILE_BYTES;

    // S = Q K^T for this warp's 16 rows x 64 keys
    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      uint32_t a[4];
      ldsm_x4(a[0], a[1], a[2], a[3], sQ + (warp * 16 + (lane & 15)) * C::ROW_BYTES + (ks * 16 + (lane >> 4) * 8) * 2);
#pragma unroll
      for (int nt = 0; nt < 8; nt += 2) {
        uint32_t b0, b1, b2, b3;
        const int mi = lane >> 3, r = lane & 7;
        ldsm_x4(b0, b1, b2, b3, sK + ((nt + (mi >> 1)) * 8 + r) * C::ROW_BYTES + (ks * 16 + (mi & 1) * 8) * 2);
        mma_bf16_16816(s[nt], a, b0, b1);
        mma_bf16_16816(s[nt + 1], a, b2, b3);
      }
    }
    // mask, scale, online softmax
    float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = blk * 64 + nt * 8 + tq * 2 + (e & 1);
        const int i = qrow[e >> 1];
        const bool vis = j < p.n_keys &&
                         (j < valid_prefix || (j >= p.prefix_alloc && (i >= p.restrict_rows || j <= p.prefix_alloc)));
        const float x = vis ? s[nt][e] * p.scale_log2e : -1e30f;
        s[nt][e] = x;
        m_new[e >> 1] = fmaxf(m_new[e >> 1], x);
      }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 1));
      m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 2));
    }
    float corr[2], l_add[2] = {0.f, 0.f};
#pragma unroll
    for (int h = 0; h < 2; ++h) corr[h] = exp2f(m_run[h] - m_new[h]);
    uint32_t pa[4][4];   // probabilities as A fragments: 4 k-steps of 16 keys
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      float e0 = s[nt][0] > -1e29f ? exp2f(s[nt][0] - m_new[0]) : 0.f;
      float e1 = s[nt][1] > -1e29f ? exp2f(s[nt][1] - m_new[0]) : 0.f;
      float e2 = s[nt][2] > -1e29f ? exp2f(s[nt][2] - m_new[1]) : 0.f;
      float e3 = s[nt][3] > -1e29f ? exp2f(s[nt][3] - m_new[1]) : 0.f;
      l_add[0] += e0 + e1;
      l_add[1] += e2 + e3;
      pa[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16(e0, e1);
      pa[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(e2, e3);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      l_run[h] = l_run[h] * corr[h] + l_add[h];
      m_run[h] = m_new[h];
    }
#pragma unroll
    for (int dt = 0; dt < DT; ++dt) {
      acc[dt][0] *= corr[0]; acc[dt][1] *= corr[0];
      acc[dt][2] *= corr[1]; acc[dt][3] *= corr[1];
    }
    // O += P V
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
      for (int dt = 0; dt < DT; dt += 2) {
        uint32_t b0, b1, b2, b3;
        const int mi = lane >> 3, r = lane & 7;
        ldsm_x4_t(b0, b1, b2, b3, sV + (kk * 16 + (mi & 1) * 8 + r) * C::ROW_BYTES + ((dt + (mi >> 1)) * 8) * 2);
        mma_bf16_16816(acc[dt], pa[kk], b0, b1);
        mma_bf16_16816(acc[dt + 1], pa[kk], b2, b3);
      }
    }
    __syncthreads();   // all warps done with this K/V buffer before it is refilled
  }
  if (blk_begin >= blk_end) cp_async_wait<0>();

  // full row sums (each quad holds partial sums of its 2 rows)
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }

  if (ksplit == 1) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int i = qrow[h];
      if (i >= p.n_q) continue;
      const float inv = l_run[h] > 0.f ? 1.f / l_run[h] : 0.f;
#pragma unroll
      for (int dt = 0; dt < DT; ++dt) {
        const int d = dt * 8 + tq * 2;
        if (d < HD)
          *reinterpret_cast<uint32_t*>(O + (size_t)i * p.ldo + d) = pack_bf16(acc[dt][h * 2] * inv, acc[dt][h * 2 + 1] * inv);
      }
    }
    KTRACE(22);
    return;
  }

  // ---- merge the key splits: partial (O, max, sum) through a global scratch that stays in L2 ----
  // layout per cluster: [rank][64 rows][HDP + 4] floats, row = HDP outputs then (max, sum, -, -)
  constexpr int ROWF = C::HDP + 4;
  float* cl_scratch = p.scratch + ((size_t)blockIdx.z * gridDim.y + blockIdx.y) * ksplit * 64 * ROWF;
  {
    float* mine = cl_scratch + (size_t)rank * 64 * ROWF;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int lr = warp * 16 + g + h * 8;
#pragma unroll
      for (int dt = 0; dt < DT; ++dt)
        __stcg(reinterpret_cast<float2*>(mine + lr * ROWF + dt * 8 + tq * 2), make_float2(acc[dt][h * 2], acc[dt][h * 2 + 1]));
      if (tq == 0) __stcg(reinterpret_cast<float2*>(mine + lr * ROWF + C::HDP), make_float2(m_run[h], l_run[h]));
    }
  }
  cluster_sync_all();   // release/acquire at cluster scope: all partials of the cluster are visible
  {
    // this CTA finishes the head-dim slice [d_begin, d_end) of all 64 rows, 4 columns per thread and step
    const int d_begin = (int)(((long long)rank * C::HDP) / ksplit) & ~3;
    const int d_end = rank == ksplit - 1 ? C::HDP : ((int)(((long long)(rank + 1) * C::HDP) / ksplit) & ~3);
    const int width = (d_end - d_begin) >> 2;          // float4 groups
    for (int idx = threadIdx.x; idx < 64 * width; idx += 128) {
      const int lr = idx / width, d = d_begin + (idx - lr * width) * 4;
      const int i = row0 + lr;
      if (i >= p.n_q) continue;
      float2 ml[8];
      float4 a[8];
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        if (r < ksplit) {
          const float* src = cl_scratch + ((size_t)r * 64 + lr) * ROWF;
          ml[r] = __ldcg(reinterpret_cast<const float2*>(src + C::HDP));
          a[r] = __ldcg(reinterpret_cast<const float4*>(src + d));
        }
      }
      float m_tot = -1e30f;
#pragma unroll
      for (int r = 0; r < 8; ++r)
        if (r < ksplit) m_tot = fmaxf(m_tot, ml[r].x);
      float l_tot = 0.f;
      float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        if (r < ksplit) {
          const float w = exp2f(ml[r].x - m_tot);
          l_tot += ml[r].y * w;
          o.x += a[r].x * w; o.y += a[r].y * w; o.z += a[r].z * w; o.w += a[r].w * w;
        }
      }
      const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
      if (d + 3 < HD) {
        *reinterpret_cast<uint2*>(O + (size_t)i * p.ldo + d) = make_uint2(pack_bf16(o.x * inv, o.y * inv), pack_bf16(o.z * inv, o.w * inv));
      } else {
        const float ov[4] = {o.x * inv, o.y * inv, o.z * inv, o.w * inv};
        for (int e = 0; e < 4; ++e)
          if (d + e < HD) O[(size_t)i * p.ldo + d + e] = __float2bfloat16(ov[e]);
      }
    }
  }
  KTRACE(22);
}
