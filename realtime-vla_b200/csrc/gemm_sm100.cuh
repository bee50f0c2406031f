// Weight-stationary GEMM for sm_100a: Y[token, feature] = X[token, :] . W[feature, :]  (+ fused epilogue)
//
//   A operand = weights, repacked once at load time to K-major [features, K]   (UMMA M = 128 features)
//   B operand = activations, row-major bf16 [tokens, K], i.e. K-major           (UMMA N = token tile)
//   D         = fp32 accumulator in TMEM: lane = feature, column = token
//
// One CTA computes a 128-feature x BN-token tile.  Roles: warp 0 = TMA producer, warp 1 = tcgen05.mma
// issuer (and TMEM owner), warps 2..5 = epilogue (one TMEM lane quarter each).  The K loop can be split
// over the CTAs of a thread-block cluster (cluster size = split); partial accumulators are then reduced
// through distributed shared memory in a fixed order, so results do not depend on scheduling.
// This is what lets the M=51 action-expert layers and the M=256 prefix layers put every SM on the
// weight stream.  All waits are bounded (see mbar_wait).
#pragma once
#include "common.cuh"

enum GemmEpiKind { EPI_BF16 = 0, EPI_RESID = 1, EPI_QKV = 2 };
enum GemmAct { ACT_NONE = 0, ACT_GELU = 1, ACT_SILU = 2, ACT_GEGLU = 3 };

struct GemmEpi {
  int kind;
  int act;
  const float* bias;  // [features] or null
  // EPI_BF16: out[t*ld_out + n] = bf16(act(v + bias[n]))          (ACT_GEGLU: gelu(v) * v2)
  bf16* out;
  int ld_out;
  // EPI_RESID: outf[t*ld_outf + n] = res_in[(t % res_mod)*ld_res + n] + bias[n] + gate[n] * v
  //            (res_in may alias outf for an in-place residual add; gate null = 1; res_in null = 0)
  float* outf;
  int ld_outf;
  const float* res_in;
  int res_mod;
  int ld_res;
  const float* gate;
  bf16* mirror;  // optional bf16 copy of the value written to outf
  int ld_mirror;
  int out_rpo;         // > 0: token t is written to row (t / out_rpo) * out_obs_stride + t % out_rpo
  int out_obs_stride;
  // EPI_QKV: features [0,2048) = 8 query heads, [2048,2304) = key, [2304,2560) = value (head dim 256).
  // Rotary embedding on adjacent pairs of Q and K; Q -> q[t*2048 + n]; K,V -> cache rows.
  bf16* q;
  bf16* kc;
  bf16* vc;
  const float* rope_cos;  // [pos][128]
  const float* rope_sin;
  const int* pos_base;    // optional device scalar added to the position
  int pos_off;
  int rows_per_obs;       // token t belongs to observation t / rows_per_obs, local row t % rows_per_obs
  int kv_obs_stride;      // cache rows per observation
  int kv_row_off;         // first cache row for local row 0
};

struct GemmParams {
  CUtensorMap tmA;   // weights [features_padded, Kp], box 64 x 128
  CUtensorMap tmA2;  // second weight (GeGLU "up"), only for DUAL
  CUtensorMap tmB;   // activations [tokens, K], box 64 x BN
  int n_feat;        // valid features
  int n_tok;         // valid tokens
  int k_blocks;      // Kp / 64
  int split;         // cluster size along K (1 = no cluster)
  int* status;       // device status word
  GemmEpi epi;
};

template <int BN, bool DUAL>
struct GemmCfg {
  static constexpr int A_BYTES = 128 * 64 * 2;
  static constexpr int B_BYTES = BN * 64 * 2;
  static constexpr int STAGE_BYTES = A_BYTES * (DUAL ? 2 : 1) + B_BYTES;
  static constexpr int MAX_STAGE_SMEM = 200 * 1024;
  static constexpr int STAGES_RAW = MAX_STAGE_SMEM / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int TMEM_COLS = DUAL ? 2 * BN : BN;
  static constexpr int BAR_BYTES = 256;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + BAR_BYTES + 1024;
  static constexpr int PARTIAL_BYTES = 128 * BN * 4 * (DUAL ? 2 : 1);  // split-K partial tile
  static constexpr bool CAN_SPLIT = PARTIAL_BYTES <= STAGES * STAGE_BYTES;
};

// smem matrix descriptor: K-major tile, rows of 128 B, 128-byte swizzle, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
  return (uint64_t)((smem_addr & 0x3FFFF) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

__device__ __forceinline__ void gemm_epilogue_store(const GemmEpi& e, int n, int t, float v, float v2, bool n_ok,
                                                    int n_feat) {
  if (e.kind == EPI_BF16) {
    if (!n_ok) return;
    if (e.bias) v += e.bias[n];
    if (e.act == ACT_GELU) v = gelu_tanh_f(v);
    else if (e.act == ACT_SILU) v = silu_f(v);
    else if (e.act == ACT_GEGLU) v = gelu_tanh_f(v) * v2;
    e.out[(size_t)t * e.ld_out + n] = __float2bfloat16(v);
  } else if (e.kind == EPI_RESID) {
    if (!n_ok) return;
    if (e.gate) v *= e.gate[n];
    if (e.bias) v += e.bias[n];
    const size_t orow = e.out_rpo > 0 ? (size_t)(t / e.out_rpo) * e.out_obs_stride + t % e.out_rpo : (size_t)t;
    if (e.res_in) v += e.res_in[(size_t)(e.res_mod > 0 ? t % e.res_mod : (int)orow) * e.ld_res + n];
    e.outf[orow * e.ld_outf + n] = v;
    if (e.mirror) e.mirror[orow * e.ld_mirror + n] = __float2bfloat16(v);
  } else {  // EPI_QKV
    const int obs = t / e.rows_per_obs, r = t - obs * e.rows_per_obs;
    const float partner = __shfl_xor_sync(0xffffffffu, v, 1);
    if (n < 2304) {
      const int pos = r + e.pos_off + (e.pos_base ? *e.pos_base : 0);
      const int i = (n & 255) >> 1;
      const float c = e.rope_cos[pos * 128 + i], s = e.rope_sin[pos * 128 + i];
      v = (n & 1) ? (v * c + partner * s) : (v * c - partner * s);
    }
    if (!n_ok) return;
    const bf16 o = __float2bfloat16(v);
    if (n < 2048) {
      e.q[(size_t)t * 2048 + n] = o;
    } else {
      const size_t row = (size_t)obs * e.kv_obs_stride + e.kv_row_off + r;
      if (n < 2304) e.kc[row * 256 + (n - 2048)] = o;
      else e.vc[row * 256 + (n - 2304)] = o;
    }
  }
}

template <int BN, bool DUAL>
__global__ void __launch_bounds__(192, 1) gemm_sm100_kernel(const __grid_constant__ GemmParams p) {
  using C = GemmCfg<BN, DUAL>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  const uint32_t smem_base = raw_addr + pad;

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES);
  const uint32_t full_bar = smem_base + C::STAGES * C::STAGE_BYTES;     // [STAGES]
  const uint32_t empty_bar = full_bar + 8 * C::STAGES;                  // [STAGES]
  const uint32_t tmem_full_bar = empty_bar + 8 * C::STAGES;             // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * C::STAGES + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = p.split;
  const int rank = blockIdx.x;  // == cluster rank: cluster dims are (split,1,1) and gridDim.x == split
  const int tok0 = blockIdx.y * BN;
  const int feat0 = blockIdx.z * 128;
  const int kb_begin = (int)(((long long)rank * p.k_blocks) / split);
  const int kb_end = (int)(((long long)(rank + 1) * p.k_blocks) / split);
  const int n_iters = kb_end - kb_begin;
  int umma_n = p.n_tok - tok0;
  umma_n = umma_n > BN ? BN : ((umma_n + 15) & ~15);

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(full_bar + 8 * s, 1);
      mbar_init(empty_bar + 8 * s, 1);
    }
    mbar_init(tmem_full_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&p.tmA);
    tma_prefetch_desc(&p.tmB);
    if (DUAL) tma_prefetch_desc(&p.tmA2);
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Everything above is independent of the previous kernel's output.
  pdl_wait();
  pdl_trigger();

  if (warp == 0) {
    if (lane == 0) {
      const uint64_t pol_w = policy_evict_first();
      const uint64_t pol_x = policy_evict_last();
      for (int it = 0; it < n_iters; ++it) {
        const int s = it % C::STAGES;
        const uint32_t ph = (uint32_t)(it / C::STAGES) & 1u;
        if (!mbar_wait(empty_bar + 8 * s, ph ^ 1u, abort_flag)) break;
        const uint32_t st = smem_base + s * C::STAGE_BYTES;
        const int k0 = (kb_begin + it) * 64;
        mbar_expect_tx(full_bar + 8 * s, C::STAGE_BYTES);
        tma_load_2d(st, &p.tmA, full_bar + 8 * s, k0, feat0, pol_w);
        if (DUAL) tma_load_2d(st + C::A_BYTES, &p.tmA2, full_bar + 8 * s, k0, feat0, pol_w);
        tma_load_2d(st + C::A_BYTES * (DUAL ? 2 : 1), &p.tmB, full_bar + 8 * s, k0, tok0, pol_x);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      // instruction descriptor: D=f32, A=B=bf16, both K-major, N = umma_n, M = 128
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(umma_n >> 3) << 17) | (8u << 24);
      bool ok = true;
      for (int it = 0; it < n_iters && ok; ++it) {
        const int s = it % C::STAGES;
        const uint32_t ph = (uint32_t)(it / C::STAGES) & 1u;
        ok = mbar_wait(full_bar + 8 * s, ph, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t st = smem_base + s * C::STAGE_BYTES;
        const uint64_t da = umma_desc_sw128(st);
        const uint64_t da2 = umma_desc_sw128(st + C::A_BYTES);
        const uint64_t db = umma_desc_sw128(st + C::A_BYTES * (DUAL ? 2 : 1));
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint32_t acc = (it | kk) != 0;
          umma_bf16(tmem_base, da + 2 * kk, db + 2 * kk, idesc, acc);
          if (DUAL) umma_bf16(tmem_base + BN, da2 + 2 * kk, db + 2 * kk, idesc, acc);
        }
        umma_commit(empty_bar + 8 * s);  // frees this smem stage once the MMAs have read it
      }
      if (ok) umma_commit(tmem_full_bar);
    }
    __syncwarp();
  }

  // ---------------- epilogue ----------------
  const bool is_epi = warp >= 2;
  const int q = warp & 3;                 // TMEM lane quarter this warp may read
  const int fl = q * 32 + lane;           // feature lane 0..127
  const int n = feat0 + fl;
  const bool n_ok = n < p.n_feat;
  bool acc_ok = false;
  if (is_epi) {
    acc_ok = mbar_wait(tmem_full_bar, 0, abort_flag);
    tc_fence_after();
  }
  const uint32_t t_lane = tmem_base + ((uint32_t)(q * 32) << 16);
  float* part = reinterpret_cast<float*>(smem);   // [acc][col][128] when split > 1 (reuses the stage buffers)

  if (split == 1) {
    if (is_epi && acc_ok) {
      for (int c0 = 0; c0 < umma_n; c0 += 32) {
        uint32_t v[32], v2[32];
        tmem_ld32(t_lane + c0, v);
        if (DUAL) tmem_ld32(t_lane + BN + c0, v2);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int t = tok0 + c0 + j;
          if (t < p.n_tok)
            gemm_epilogue_store(p.epi, n, t, __uint_as_float(v[j]), DUAL ? __uint_as_float(v2[j]) : 0.f, n_ok,
                                p.n_feat);
        }
      }
    }
  } else {
    if (is_epi && acc_ok) {
      for (int c0 = 0; c0 < umma_n; c0 += 32) {
        uint32_t v[32];
        tmem_ld32(t_lane + c0, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) part[(c0 + j) * 128 + fl] = __uint_as_float(v[j]);
        if (DUAL) {
          tmem_ld32(t_lane + BN + c0, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) part[(BN + c0 + j) * 128 + fl] = __uint_as_float(v[j]);
        }
      }
    }
    __syncwarp();
    cluster_sync_all();
    if (is_epi) {
      const int n_cols = min(umma_n, p.n_tok - tok0);
      const uint32_t my_part = smem_base;
      for (int c = rank; c < n_cols; c += split) {
        float s1 = 0.f, s2 = 0.f;
        for (int r = 0; r < split; ++r) {
          const uint32_t remote = dsmem_map(my_part, (uint32_t)r);
          s1 += dsmem_ld_f32(remote + (uint32_t)(c * 128 + fl) * 4u);
          if (DUAL) s2 += dsmem_ld_f32(remote + (uint32_t)((BN + c) * 128 + fl) * 4u);
        }
        gemm_epilogue_store(p.epi, n, tok0 + c, s1, s2, n_ok, p.n_feat);
      }
    }
    __syncwarp();
    cluster_sync_all();   // nobody leaves while a peer may still read its partial tile
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0 && p.status) atomicOr(p.status, VLA_ST_WAIT_TIMEOUT);
    for (int i = 0; i < 32; ++i) __nanosleep(1000);   // let any copy still in flight land before the CTA exits
  }
  if (warp == 1) tmem_dealloc(tmem_base, C::TMEM_COLS);
}
