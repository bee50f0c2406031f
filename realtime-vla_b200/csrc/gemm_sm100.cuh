// Weight-stationary GEMM for sm_100a: Y[token, feature] = X[token, :] . W[feature, :]  (+ fused epilogue)
//
//   A operand = weights, repacked once at load time to K-major [features, K]   (UMMA M = 128 features)
//   B operand = activations, row-major bf16 [tokens, K], i.e. K-major           (UMMA N = token tile)
//   D         = fp32 accumulator in TMEM: lane = feature, column = token
//
// One CTA computes a 128-feature x BN-token tile.  Roles: warp 0 = TMA producer, warp 1 = tcgen05.mma
// issuer (and TMEM owner), warps 2..9 = epilogue (two warps per TMEM lane quarter, alternating 32-column
// chunks).  The K loop can be split over the CTAs of a thread-block cluster (cluster size = split): every
// CTA then writes its fp32 partial tile to a scratch area in global memory (it stays in L2; distributed
// shared memory moves only ~15 B/clk per SM and was 3-4x slower here), one cluster barrier orders the
// writes, and the CTA that owns a column (column c belongs to rank c % split) adds the `split` partials in
// rank order, so results do not depend on scheduling.  This is what lets the M=51 action-expert layers
// and the M=256 prefix layers put every SM on the weight stream.  All mbarrier waits are bounded (see
// mbar_wait).
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
  const float* mirror_scale;  // optional [features]: the mirror holds value * (1 + mirror_scale[n]) (adaRMS scale of the
                              // norm that consumes it, pi05_infer.py:78-113: y = rms(x) * (1 + scale) + shift)
  const float* bias2;         // optional bias of the second accumulator (GeGLU "up"); with ssq_in both biases are
                              // added after the per-token scale, i.e. they carry shift @ W of a folded adaRMS norm
  int out_rpo;         // > 0: token t is written to row (t / out_rpo) * out_obs_stride + t % out_rpo
  int out_obs_stride;
  // RMS norm folded into the GEMMs around a residual stream (the normalisation has no learned scale, so
  // norm(x) @ W = f * (x @ W) with f = rsqrt(mean(x^2) + 1e-6) per token, pi0_infer.py:1005):
  float* ssq_out;      // EPI_RESID producer: sum of squares of the written values per (32-feature slot, token)
  int ssq_ld;          //   ssq_out[slot * ssq_ld + token]
  const float* ssq_in; // consumer (any kind): accumulators are scaled by f[token] from these partial sums
  int ssq_slots;       //   number of slots (= features of the normalised stream / 32)
  float ssq_inv_d;     //   1 / features
  // EPI_QKV: features [0,2048) = 8 query heads, [2048,2304) = key, [2304,2560) = value (head dim 256).
  // Rotary embedding on adjacent pairs of Q and K; Q -> q[t*2048 + n]; K,V -> cache rows.
  bf16* q;
  bf16* kc;
  bf16* vc;
  bf16* vt;               // optional transposed value cache [observation][256][vt_ld] (read by the tcgen05 attention)
  int vt_ld;
  const float* rope_cos;  // [pos][128]
  const float* rope_sin;
  const int* pos_base;    // optional device scalar added to the position
  int pos_off;
  int rows_per_obs;       // token t belongs to observation t / rows_per_obs, local row t % rows_per_obs
  int kv_obs_stride;      // cache rows per observation
  int kv_row_off;         // first cache row for local row 0
};

// Optional in-kernel timeline for development builds (-DVLA_TRACE): CTA (0,0,0) records clock64() at the
// phase boundaries into params.trace[slot].  Compiled out otherwise.
#ifdef VLA_TRACE
#define GEMM_TRACE(slot)                                                                             \
  do {                                                                                               \
    if (p.trace && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) p.trace[slot] = clock64(); \
  } while (0)
#else
#define GEMM_TRACE(slot) do {} while (0)
#endif

struct GemmParams {
  CUtensorMap tmA;   // weights [features_padded, Kp], box 64 x 128
  CUtensorMap tmA2;  // second weight (GeGLU "up"), only for DUAL
  CUtensorMap tmB;   // activations [tokens, K], box 64 x BN
  CUtensorMap tmOut; // output [tokens, features], box 32 x 32, no swizzle (see out_mode); QKV: the query buffer
  CUtensorMap tmOut2; // QKV only: key cache rows [kv_row_off + tokens, 256]
  CUtensorMap tmOut3; // QKV only: value cache rows
  int out_mode;      // 0: epilogue stores with plain st.global; 1: bf16 tile stores through TMA; 2: fp32 tile stores;
                     // 3: fp32 tile reduce-add (in-place residual: x += gate*acc + bias, one add per element);
                     // 4: QKV with rotary embedding, bf16 tile stores into the query buffer and the K/V cache
  int n_feat;        // valid features
  int n_tok;         // valid tokens
  int k_blocks;      // Kp / 64
  int split;         // cluster size along K (1 = no cluster)
  int tok_tile;      // tokens per CTA along grid.y, a multiple of 32 and <= BN (0 = BN): the host evens the tiles out
                     // (788 tokens = 4 x 224 rather than 3 x 256 + 20) so that the last tile does not stream the
                     // whole weight panel for a handful of tokens; the B box of tmB has this many rows
  int cg2;           // launch of the CG2 variant (tcgen05 CTA pairs): gridDim.x = 2 * split, gridDim.z = pairs of feature
                     // tiles, the B box of tmB has tok_tile / 2 rows
  int m256;          // launch of the PAIR variant: the two accumulators are two feature tiles of ONE weight
                     // (features feat0.. and feat0+128..) instead of the gate/up pair; each gets the plain epilogue
  int* status;       // device status word
  float* scratch;    // split-K partial tiles: [tile][src rank][accumulator][column][128 features] fp32
  long long* trace;  // development timeline (see GEMM_TRACE), normally null
  GemmEpi epi;
};

constexpr int GEMM_THREADS = 320;

// SPLITK variants are launched as clusters of `split` CTAs along K.  CG2 variants run as tcgen05 CTA pairs: two
// CTAs on neighbouring feature tiles share one activation tile, of which each loads half (see the kernel).
template <int BN, bool DUAL, bool SPLITK, bool CG2 = false>
struct GemmCfg {
  static constexpr int A_BYTES = 128 * 64 * 2;
  static constexpr int B_BYTES = (CG2 ? BN / 2 : BN) * 64 * 2;
  static constexpr int STAGE_BYTES = A_BYTES * (DUAL ? 2 : 1) + B_BYTES;
  static constexpr int RECV_BYTES = 0;
  static constexpr int PARTIAL_FLOATS = 128 * BN * (DUAL ? 2 : 1);   // scratch floats per CTA
  static constexpr int MAX_SMEM = 204 * 1024;
  static constexpr int STAGES_RAW = (MAX_SMEM - RECV_BYTES) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : (STAGES_RAW < 1 ? 1 : STAGES_RAW);
  static constexpr bool VALID = STAGES_RAW >= 3;
  static constexpr int TMEM_COLS = DUAL ? 2 * BN : BN;
  static constexpr int BAR_BYTES = 256 + 1024;   // barriers + TMEM slot, then per-token row scales [256]
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + RECV_BYTES + BAR_BYTES + 1024;
};

// smem matrix descriptor: K-major tile, rows of 128 B, 128-byte swizzle, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
  return (uint64_t)((smem_addr & 0x3FFFF) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

__device__ __forceinline__ uint32_t pack2_bf16(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Per-thread epilogue constants (this thread owns feature n for every token column of the tile).
struct EpiThread {
  int n;
  bool n_ok;
  float bias, gate;
  float bias2, mscale;
  int pos_base;
};

// Applies the epilogue to NC accumulator columns of one feature: column j is token t0 + j*tstride, the
// first n_valid columns are real (n_valid is uniform over the warp).  The arithmetic of all columns is
// written as independent chains, and all global loads of the group are issued before the first store, so
// they overlap instead of forming a load->store->load chain (outputs may alias the residual input).
template <int NC>
__device__ __forceinline__ void gemm_epilogue_cols(const GemmEpi& e, const EpiThread& th, int t0, int tstride, int n_valid,
                                                   const float* v, const float* v2) {
  const int n = th.n;
  if (e.kind == EPI_BF16) {
    if (!th.n_ok) return;
    float x[NC];
    if (e.act == ACT_GEGLU) {
#pragma unroll
      for (int j = 0; j < NC; ++j) x[j] = gelu_tanh_f(v[j] + th.bias) * (v2[j] + th.bias2);
    } else if (e.act == ACT_GELU) {
#pragma unroll
      for (int j = 0; j < NC; ++j) x[j] = gelu_tanh_f(v[j] + th.bias);
    } else if (e.act == ACT_SILU) {
#pragma unroll
      for (int j = 0; j < NC; ++j) x[j] = silu_f(v[j] + th.bias);
    } else {
#pragma unroll
      for (int j = 0; j < NC; ++j) x[j] = v[j] + th.bias;
    }
    bf16* o = e.out + (size_t)t0 * e.ld_out + n;
    const size_t step = (size_t)tstride * e.ld_out;
#pragma unroll
    for (int j = 0; j < NC; ++j)
      if (j < n_valid) o[j * step] = __float2bfloat16(x[j]);
  } else if (e.kind == EPI_RESID) {
    // Row bookkeeping without per-column integer division (an emulated division per column made this epilogue
    // 3x slower than its memory traffic): one division for the first column, then incremental wrap-around.
    float r[NC];
    size_t orow[NC];
    int o_obs = 0, o_r = t0, m_r = t0;
    if (e.out_rpo > 0 && t0 >= e.out_rpo) { o_obs = t0 / e.out_rpo; o_r = t0 - o_obs * e.out_rpo; }
    if (e.res_mod > 0 && t0 >= e.res_mod) m_r = t0 % e.res_mod;
#pragma unroll
    for (int j = 0; j < NC; ++j) {
      orow[j] = e.out_rpo > 0 ? (size_t)o_obs * e.out_obs_stride + o_r : (size_t)(t0 + j * tstride);
      r[j] = 0.f;
      if (j < n_valid && th.n_ok && e.res_in) r[j] = e.res_in[(e.res_mod > 0 ? (size_t)m_r : orow[j]) * e.ld_res + n];
      if (e.out_rpo > 0) {
        o_r += tstride;
        if (o_r >= e.out_rpo) { o_r -= e.out_rpo; ++o_obs; }
      }
      if (e.res_mod > 0) {
        m_r += tstride;
        if (m_r >= e.res_mod) m_r -= e.res_mod;
      }
    }
#pragma unroll
    for (int j = 0; j < NC; ++j) r[j] += v[j] * th.gate + th.bias;
#pragma unroll
    for (int j = 0; j < NC; ++j) {
      if (j < n_valid && th.n_ok) {
        e.outf[orow[j] * e.ld_outf + n] = r[j];
        if (e.mirror) e.mirror[orow[j] * e.ld_mirror + n] = __float2bfloat16(r[j] * th.mscale);
      }
    }
    if (e.ssq_out) {   // per-token sum of squares over this warp's 32 features (warp-collective: no early exit above)
#pragma unroll
      for (int j = 0; j < NC; ++j) {
        float sq = (j < n_valid && th.n_ok) ? r[j] * r[j] : 0.f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        if ((threadIdx.x & 31) == 0 && j < n_valid) e.ssq_out[(size_t)(n >> 5) * e.ssq_ld + orow[j]] = sq;
      }
    }
  } else {  // EPI_QKV
    float c[NC], s[NC];
    int lrow[NC], lobs[NC];
    const int i = (n & 255) >> 1;
    const bool rot = n < 2304;
    int obs = 0, rr = t0;
    if (t0 >= e.rows_per_obs) { obs = t0 / e.rows_per_obs; rr = t0 - obs * e.rows_per_obs; }
#pragma unroll
    for (int j = 0; j < NC; ++j) {
      lrow[j] = rr;
      lobs[j] = obs;
      c[j] = 1.f;
      s[j] = 0.f;
      if (j < n_valid && rot) {
        const int pos = rr + e.pos_off + th.pos_base;
        c[j] = e.rope_cos[pos * 128 + i];
        s[j] = e.rope_sin[pos * 128 + i];
      }
      rr += tstride;
      if (rr >= e.rows_per_obs) { rr -= e.rows_per_obs; ++obs; }
    }
    const float sgn = (n & 1) ? 1.f : -1.f;
    float x[NC];
#pragma unroll
    for (int j = 0; j < NC; ++j) {
      const float val = v[j] + th.bias;
      const float partner = __shfl_xor_sync(0xffffffffu, val, 1);
      x[j] = val * c[j] + sgn * partner * s[j];
    }
#pragma unroll
    for (int j = 0; j < NC; ++j) {
      if (j < n_valid) {
        const bf16 o = __float2bfloat16(x[j]);
        if (n < 2048) {
          e.q[(size_t)(t0 + j * tstride) * 2048 + n] = o;
        } else {
          const size_t row = (size_t)lobs[j] * e.kv_obs_stride + e.kv_row_off + lrow[j];
          if (n < 2304) e.kc[row * 256 + (n - 2048)] = o;
          else {
            e.vc[row * 256 + (n - 2304)] = o;
            if (e.vt) e.vt[((size_t)lobs[j] * 256 + (n - 2304)) * e.vt_ld + e.kv_row_off + lrow[j]] = o;
          }
        }
      }
    }
  }
}

// DUAL: gate/up pair of two weights (GeGLU).  PAIR: two 128-feature tiles of one weight, each with the plain
// epilogue.  Both keep two accumulators that share the activation tile (TWO).
// CG2: the CTAs with blockIdx.x = 2 r and 2 r + 1 (neighbours in the cluster) form a tcgen05 CTA pair on the feature
// tiles 2 z and 2 z + 1 of the same token tile and K slice r: each CTA brings in its own 128 x 64 weight tile and HALF of
// the activation tile (the per-SM L2 read rate, ~60 B/clk, bounds a single CTA's 128 x 256 tile at 2/3 of the MMA
// rate; the pair needs 2/3 of the bytes per MMA cycle), every load completes on the even CTA's barrier, whose MMA thread
// issues cta_group::2 MMAs of M = 256 for both, and each CTA runs the unchanged epilogue on its own 128 accumulator rows.
template <int BN, bool DUAL, bool SPLITK, bool PAIR = false, bool CG2 = false>
__global__ void __launch_bounds__(GEMM_THREADS, 1) gemm_sm100_kernel(const __grid_constant__ GemmParams p) {
  static_assert(!(DUAL && PAIR), "a paired launch has one weight");
  static_assert(!(CG2 && PAIR), "CTA pairs take one feature tile per CTA");
  constexpr bool TWO = DUAL || PAIR;
  constexpr bool m256 = PAIR;
  using C = GemmCfg<BN, TWO, SPLITK, CG2>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  const uint32_t smem_base = raw_addr + pad;

  constexpr int PIPE_BYTES = C::STAGES * C::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + PIPE_BYTES + C::RECV_BYTES);
  const uint32_t full_bar = smem_base + PIPE_BYTES + C::RECV_BYTES;       // [STAGES]
  const uint32_t empty_bar = full_bar + 8 * C::STAGES;                    // [STAGES]
  const uint32_t tmem_full_bar = empty_bar + 8 * C::STAGES;               // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * C::STAGES + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  KTRACE(10);
  if (threadIdx.x == 0) GEMM_TRACE(0);
  const int split = SPLITK ? p.split : 1;
  // cluster dims are (gridDim.x,1,1): blockIdx.x is the cluster rank = K slice, or 2 * K slice + rank in the CTA pair
  const int pr = CG2 ? (int)(blockIdx.x & 1u) : 0;
  const int rank = SPLITK ? (int)(CG2 ? blockIdx.x >> 1 : blockIdx.x) : 0;
  const int tok_tile = p.tok_tile > 0 ? p.tok_tile : BN;
  const int tok0 = blockIdx.y * tok_tile;
  // bytes one K block brings in (CG2: both CTAs' weight tiles and halves of the activation tile, counted by the leader)
  const uint32_t stage_tx = CG2 ? (uint32_t)(2 * (C::A_BYTES * (TWO ? 2 : 1) + (tok_tile / 2) * 128))
                                : (uint32_t)(C::A_BYTES * (TWO ? 2 : 1) + tok_tile * 128);
  const int feat_tile = CG2 ? (int)blockIdx.z * 2 + pr : (int)blockIdx.z;
  const int feat0 = feat_tile * (m256 ? 256 : 128);
  const int kb_begin = (int)(((long long)rank * p.k_blocks) / split);
  const int kb_end = (int)(((long long)(rank + 1) * p.k_blocks) / split);
  const int n_iters = kb_end - kb_begin;
  int umma_n = p.n_tok - tok0;
  umma_n = umma_n > tok_tile ? tok_tile : ((umma_n + 15) & ~15);

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
    if (p.out_mode) tma_prefetch_desc(&p.tmOut);
    if (p.out_mode == 4) { tma_prefetch_desc(&p.tmOut2); tma_prefetch_desc(&p.tmOut3); }
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) GEMM_TRACE(1);
  // CTA pair: the peer's barriers must exist before anything signals them, and one MMA addresses the accumulators of
  // both CTAs with one tensor-memory address, so the two allocations must have returned the same one (they do when each
  // SM holds one CTA with tensor memory at a time; otherwise the launch gives up and says so in the status word).
  uint32_t full_bar_lead = full_bar;   // shared::cluster address of the leader's full barriers
  if (CG2) {
    cluster_sync_all();
    const uint32_t my_rank = cluster_ctarank();
    full_bar_lead = dsmem_map(full_bar, my_rank & ~1u);
    const uint32_t peer_base = dsmem_ld_u32(dsmem_map(smem_u32(tmem_slot), my_rank ^ 1u));
    if (peer_base != tmem_base) {
      if (threadIdx.x == 0) {
        *abort_flag = 1;
        if (p.status) atomicOr(p.status, VLA_ST_BAD_SHAPE);
      }
    }
    __syncthreads();
  }
  const bool pair_ok = !CG2 || *abort_flag == 0;

  // Let the next kernels of the stream start now: their prologue and weight prefetch run under this kernel
  // (they block in their own griddepcontrol.wait until this grid has completed).
  pdl_trigger();
  // Weights do not depend on the previous kernel: fill the pipeline with weight tiles before waiting for it.
  const int n_pre = n_iters < C::STAGES ? n_iters : C::STAGES;
  uint64_t pol_w = 0;
  if (warp == 0 && lane == 0 && pair_ok) {
    pol_w = policy_evict_first();
    for (int it = 0; it < n_pre; ++it) {
      const uint32_t st = smem_base + it * C::STAGE_BYTES;
      const int k0 = (kb_begin + it) * 64;
      if (pr == 0) mbar_expect_tx(full_bar + 8 * it, stage_tx);
      if (CG2) {
        tma_load_2d_pair(st, &p.tmA, full_bar_lead + 8 * it, k0, feat0, pol_w);
        if (TWO) tma_load_2d_pair(st + C::A_BYTES, &p.tmA2, full_bar_lead + 8 * it, k0, feat0, pol_w);
      } else {
        tma_load_2d(st, &p.tmA, full_bar + 8 * it, k0, feat0, pol_w);
        if (TWO) tma_load_2d(st + C::A_BYTES, m256 ? &p.tmA : &p.tmA2, full_bar + 8 * it, k0, feat0 + (m256 ? 128 : 0), pol_w);
      }
    }
  }
  // Activations (and everything the epilogue reads or writes) do.
  pdl_wait();
  KTRACE(11);
  if (threadIdx.x == 0) GEMM_TRACE(2);

  if (warp == 0) {
    if (lane == 0 && pair_ok) {
      const uint64_t pol_x = policy_evict_last();
      const int tok_b = CG2 ? tok0 + pr * (umma_n >> 1) : tok0;   // CTA pair: rows [0, N/2) and [N/2, N) of the tile
      for (int it = 0; it < n_iters; ++it) {
        const int s = it % C::STAGES;
        const uint32_t st = smem_base + s * C::STAGE_BYTES;
        const int k0 = (kb_begin + it) * 64;
        if (it >= n_pre) {
          const uint32_t ph = (uint32_t)(it / C::STAGES) & 1u;
          if (!mbar_wait(empty_bar + 8 * s, ph ^ 1u, abort_flag)) break;
          if (pr == 0) mbar_expect_tx(full_bar + 8 * s, stage_tx);
          if (CG2) {
            tma_load_2d_pair(st, &p.tmA, full_bar_lead + 8 * s, k0, feat0, pol_w);
            if (TWO) tma_load_2d_pair(st + C::A_BYTES, &p.tmA2, full_bar_lead + 8 * s, k0, feat0, pol_w);
          } else {
            tma_load_2d(st, &p.tmA, full_bar + 8 * s, k0, feat0, pol_w);
            if (TWO) tma_load_2d(st + C::A_BYTES, m256 ? &p.tmA : &p.tmA2, full_bar + 8 * s, k0, feat0 + (m256 ? 128 : 0), pol_w);
          }
        }
        if (CG2) tma_load_2d_pair(st + C::A_BYTES * (TWO ? 2 : 1), &p.tmB, full_bar_lead + 8 * s, k0, tok_b, pol_x);
        else tma_load_2d(st + C::A_BYTES * (TWO ? 2 : 1), &p.tmB, full_bar + 8 * s, k0, tok0, pol_x);
      }
      GEMM_TRACE(3);
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0 && pr == 0 && pair_ok) {
      // instruction descriptor: D=f32, A=B=bf16, both K-major, N = umma_n, M = 128 (256 over a CTA pair)
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(umma_n >> 3) << 17) | ((CG2 ? 16u : 8u) << 24);
      const uint16_t pair_mask = (uint16_t)(3u << (CG2 ? (cluster_ctarank() & ~1u) : 0u));
      bool ok = true;
      for (int it = 0; it < n_iters && ok; ++it) {
        const int s = it % C::STAGES;
        const uint32_t ph = (uint32_t)(it / C::STAGES) & 1u;
        ok = mbar_wait(full_bar + 8 * s, ph, abort_flag);
        if (!ok) break;
        tc_fence_after();
        if (it == 0) GEMM_TRACE(4);
        if (it == 0) KTRACE_T(17, 32);
        const uint32_t st = smem_base + s * C::STAGE_BYTES;
        const uint64_t da = umma_desc_sw128(st);
        const uint64_t da2 = umma_desc_sw128(st + C::A_BYTES);
        const uint64_t db = umma_desc_sw128(st + C::A_BYTES * (TWO ? 2 : 1));
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint32_t acc = (it | kk) != 0;
          if (CG2) {
            umma_bf16_pair(tmem_base, da + 2 * kk, db + 2 * kk, idesc, acc);
            if (TWO) umma_bf16_pair(tmem_base + BN, da2 + 2 * kk, db + 2 * kk, idesc, acc);
          } else {
            umma_bf16(tmem_base, da + 2 * kk, db + 2 * kk, idesc, acc);
            if (TWO) umma_bf16(tmem_base + BN, da2 + 2 * kk, db + 2 * kk, idesc, acc);
          }
        }
        // frees this smem stage (in both CTAs of a pair) once the MMAs have read it
        if (CG2) umma_commit_pair(empty_bar + 8 * s, pair_mask);
        else umma_commit(empty_bar + 8 * s);
      }
      if (ok) {
        if (CG2) umma_commit_pair(tmem_full_bar, pair_mask);
        else umma_commit(tmem_full_bar);
      }
      GEMM_TRACE(5);
    }
    __syncwarp();
  }

  // ---------------- epilogue ----------------
  const bool is_epi = warp >= 2;
  float* row_scale = reinterpret_cast<float*>(smem + PIPE_BYTES + 256);   // [BN] when the RMS norm is folded in
  const bool scaled = p.epi.ssq_in != nullptr;
  if (is_epi && scaled) {
    // 256 epilogue threads, one token each: f = rsqrt(mean(x^2) + eps) from the producer's partial sums
    const int tt = threadIdx.x - 64;
    if (tt < umma_n) {
      const int t = min(tok0 + tt, p.n_tok - 1);
      float acc = 0.f;
      for (int sl = 0; sl < p.epi.ssq_slots; ++sl) acc += p.epi.ssq_in[(size_t)sl * p.epi.ssq_ld + t];
      row_scale[tt] = rsqrtf(acc * p.epi.ssq_inv_d + 1e-6f);
    }
    asm volatile("bar.sync 1, 256;" ::: "memory");   // the eight epilogue warps
  }
  const int q = warp & 3;                 // TMEM lane quarter this warp may read
  const int half = (warp - 2) >> 2;       // the two warps of a quarter take alternate column chunks
  const int fl = q * 32 + lane;           // feature lane 0..127
  const int n = feat0 + fl;
  const bool n_ok = n < p.n_feat;
  EpiThread th_first;   // per-feature constants, fetched while the main loop runs
  th_first.n = n;
  th_first.n_ok = n_ok;
  th_first.bias = (is_epi && n_ok && p.epi.bias) ? p.epi.bias[n] : 0.f;
  th_first.gate = (is_epi && n_ok && p.epi.gate) ? p.epi.gate[n] : 1.f;
  th_first.pos_base = (p.epi.kind == EPI_QKV && p.epi.pos_base) ? *p.epi.pos_base : 0;
  th_first.bias2 = (is_epi && n_ok && p.epi.bias2) ? p.epi.bias2[n] : 0.f;
  th_first.mscale = (is_epi && n_ok && p.epi.mirror_scale) ? 1.f + p.epi.mirror_scale[n] : 1.f;
  EpiThread th2 = th_first;   // second feature tile of an m256 launch
  if (m256) {
    th2.n = n + 128;
    th2.n_ok = th2.n < p.n_feat;
    th2.bias = (is_epi && th2.n_ok && p.epi.bias) ? p.epi.bias[th2.n] : 0.f;
    th2.gate = (is_epi && th2.n_ok && p.epi.gate) ? p.epi.gate[th2.n] : 1.f;
    th2.mscale = (is_epi && th2.n_ok && p.epi.mirror_scale) ? 1.f + p.epi.mirror_scale[th2.n] : 1.f;
  }
  const int n_pass = m256 ? 2 : 1;
  bool acc_ok = false;
  if (is_epi) {
    acc_ok = __all_sync(0xffffffffu, mbar_wait(tmem_full_bar, 0, abort_flag));   // TMEM loads are warp-collective
    tc_fence_after();
    if (threadIdx.x == 64) GEMM_TRACE(6);
    KTRACE_T(13, 64);
  }
  const uint32_t t_lane = tmem_base + ((uint32_t)(q * 32) << 16);

  if (!SPLITK || split == 1) {
    if (is_epi && acc_ok && p.out_mode != 0) {
      // Tile stores through TMA: each warp stages a 32-token x 32-feature block in shared memory (the pipeline
      // stages are free once the accumulator is complete) and one lane hands it to the TMA unit, which also
      // clips the rows/columns beyond the tensor.  Scattered 2- and 4-byte st.global from the thread-per-
      // feature layout cost ~30 cycles per instruction and dominated the epilogue of the large tiles.
      const bool f32 = p.out_mode == 2 || p.out_mode == 3;
      uint8_t* stg = smem + (warp - 2) * 8192;              // two 4 KB slots per warp
      const uint32_t stg_addr = smem_base + (warp - 2) * 8192;
      int it = 0;
#pragma unroll 1
      for (int pass = 0; pass < n_pass; ++pass) {
      const EpiThread& th = pass ? th2 : th_first;
      const int n = th.n;
      const int x0 = feat0 + pass * 128 + q * 32;
      for (int c0 = 32 * half; c0 < umma_n; c0 += 64, ++it) {
        uint32_t v[32], v2[32];
        if (threadIdx.x == 64 && c0 == 0) GEMM_TRACE(7);
        tmem_ld32(t_lane + pass * BN + c0, v);
        if (DUAL) tmem_ld32(t_lane + BN + c0, v2);
        tmem_ld_wait();
        if (threadIdx.x == 64 && c0 == 0) GEMM_TRACE(8);
        if (scaled) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            v[j] = __float_as_uint(__uint_as_float(v[j]) * row_scale[c0 + j]);
            if (DUAL) v2[j] = __float_as_uint(__uint_as_float(v2[j]) * row_scale[c0 + j]);
          }
        }
        const int slot = it & 1;
        if (it >= 2) {   // the store issued two chunks ago must have finished reading this slot
          if (lane == 0) bulk_wait_read<1>();
          __syncwarp();
        }
        float x[32];
        if (p.epi.kind == EPI_BF16) {
          if (p.epi.act == ACT_GEGLU) {
#pragma unroll
            for (int j = 0; j < 32; ++j) x[j] = gelu_tanh_f(__uint_as_float(v[j]) + th.bias) * (__uint_as_float(v2[j]) + th.bias2);
          } else if (p.epi.act == ACT_GELU) {
#pragma unroll
            for (int j = 0; j < 32; ++j) x[j] = gelu_tanh_f(__uint_as_float(v[j]) + th.bias);
          } else if (p.epi.act == ACT_SILU) {
#pragma unroll
            for (int j = 0; j < 32; ++j) x[j] = silu_f(__uint_as_float(v[j]) + th.bias);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) x[j] = __uint_as_float(v[j]) + th.bias;
          }
        } else if (p.epi.kind == EPI_QKV) {
          // rotary embedding on adjacent feature pairs (lanes 2i, 2i+1) of Q and K; single observation: row = token
          const bool rot = n < 2304;
          const int fi = (n & 255) >> 1;
          const float sgn = (n & 1) ? 1.f : -1.f;
          float cs[32], sn[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int pos = min(tok0 + c0 + j, p.n_tok - 1) + p.epi.pos_off + th.pos_base;
            cs[j] = rot ? p.epi.rope_cos[pos * 128 + fi] : 1.f;
            sn[j] = rot ? p.epi.rope_sin[pos * 128 + fi] : 0.f;
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float val = __uint_as_float(v[j]) + th.bias;
            const float partner = __shfl_xor_sync(0xffffffffu, val, 1);
            x[j] = val * cs[j] + sgn * partner * sn[j];
          }
          if (n >= 2304 && p.epi.vt) {   // transposed value cache: this thread owns row d, 32 consecutive keys
            bf16* dst = p.epi.vt + (size_t)(n - 2304) * p.epi.vt_ld + p.epi.kv_row_off + tok0 + c0;
            const bool vec = (((size_t)(p.epi.kv_row_off + tok0 + c0) | (size_t)p.epi.vt_ld) & 7) == 0 && tok0 + c0 + 32 <= p.n_tok;
            if (vec) {
#pragma unroll
              for (int g = 0; g < 4; ++g)
                *reinterpret_cast<uint4*>(dst + 8 * g) =
                    make_uint4(pack2_bf16(x[8 * g], x[8 * g + 1]), pack2_bf16(x[8 * g + 2], x[8 * g + 3]),
                               pack2_bf16(x[8 * g + 4], x[8 * g + 5]), pack2_bf16(x[8 * g + 6], x[8 * g + 7]));
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (tok0 + c0 + j < p.n_tok) dst[j] = __float2bfloat16(x[j]);
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) x[j] = __uint_as_float(v[j]) * th.gate + th.bias;
        }
        if (f32) {
          float* d = reinterpret_cast<float*>(stg + slot * 4096) + lane;
#pragma unroll
          for (int j = 0; j < 32; ++j) d[j * 32] = x[j];
        } else {
          bf16* d = reinterpret_cast<bf16*>(stg + slot * 4096) + lane;
#pragma unroll
          for (int j = 0; j < 32; ++j) d[j * 32] = __float2bfloat16(x[j]);
        }
        fence_proxy_async_shared();
        __syncwarp();
        if (lane == 0) {
          if (x0 < p.n_feat) {
            if (p.out_mode == 3) tma_reduce_add_2d(&p.tmOut, stg_addr + slot * 4096, x0, tok0 + c0);
            else if (p.out_mode == 4 && x0 >= 2304) tma_store_2d(&p.tmOut3, stg_addr + slot * 4096, x0 - 2304, p.epi.kv_row_off + tok0 + c0);
            else if (p.out_mode == 4 && x0 >= 2048) tma_store_2d(&p.tmOut2, stg_addr + slot * 4096, x0 - 2048, p.epi.kv_row_off + tok0 + c0);
            else tma_store_2d(&p.tmOut, stg_addr + slot * 4096, x0, tok0 + c0);
          }
          // one group per chunk even when nothing is stored (feature padding, the empty second tile of a paired
          // launch): the slot reuse above counts groups
          bulk_commit();
        }
        if (threadIdx.x == 64 && c0 == 0) GEMM_TRACE(9);
      }
      }
      if (lane == 0) bulk_wait_all();
      __syncwarp();
    } else if (is_epi && acc_ok) {
      const bool vt_by_keys = p.epi.kind == EPI_QKV && p.epi.vt != nullptr && feat0 >= 2304;
#pragma unroll 1
      for (int pass = 0; pass < n_pass; ++pass) {
        for (int c0 = 32 * half; c0 < umma_n; c0 += 64) {
          uint32_t v[32], v2[32];
          tmem_ld32(t_lane + pass * BN + c0, v);
          if (DUAL) tmem_ld32(t_lane + BN + c0, v2);
          tmem_ld_wait();
          if (scaled) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              v[j] = __float_as_uint(__uint_as_float(v[j]) * row_scale[c0 + j]);
              if (DUAL) v2[j] = __float_as_uint(__uint_as_float(v2[j]) * row_scale[c0 + j]);
            }
          }
          const int n_valid = min(32, p.n_tok - (tok0 + c0));
          if (vt_by_keys) {
            // Value tile with a transposed cache: a thread owns one feature, so writing V^T[feature][key] from the
            // accumulator layout puts the 32 lanes of a store on 32 different rows (32 partial sectors per
            // instruction; the value tiles were the long pole of the batched QKV launch).  The 32 x 32 block goes
            // through this warp's slice of the idle pipeline stages instead and is written with lanes along the keys.
            bf16* tsp = reinterpret_cast<bf16*>(smem + (warp - 2) * 8192);
            const EpiThread& th = pass ? th2 : th_first;
#pragma unroll
            for (int j = 0; j < 32; ++j) tsp[j * 34 + lane] = __float2bfloat16(__uint_as_float(v[j]) + th.bias);
            __syncwarp();
            const int t = tok0 + c0 + lane;
            if (t < p.n_tok) {
              const int obs = t / p.epi.rows_per_obs, lrow = t - obs * p.epi.rows_per_obs;
              bf16* dst = p.epi.vt + ((size_t)obs * 256 + (feat0 + pass * 128 - 2304 + q * 32)) * p.epi.vt_ld + p.epi.kv_row_off + lrow;
#pragma unroll
              for (int f = 0; f < 32; ++f) dst[(size_t)f * p.epi.vt_ld] = tsp[lane * 34 + f];
            }
            __syncwarp();
            GemmEpi e2 = p.epi;
            e2.vt = nullptr;   // the row-major value cache is written by the generic path
            gemm_epilogue_cols<32>(e2, th, tok0 + c0, 1, n_valid, reinterpret_cast<const float*>(v),
                                   reinterpret_cast<const float*>(m256 ? v : v2));
            continue;
          }
          gemm_epilogue_cols<32>(p.epi, pass ? th2 : th_first, tok0 + c0, 1, n_valid, reinterpret_cast<const float*>(v),
                                 reinterpret_cast<const float*>(m256 ? v : v2));
        }
      }
    }
  } else {
    constexpr int ACCS = TWO ? 2 : 1;
    const int n_cols = min(umma_n, p.n_tok - tok0);
    // scratch of this cluster: [src rank][accumulator][column][128 features]
    float* tile_scratch = p.scratch + (size_t)(feat_tile * gridDim.y + blockIdx.y) * split * C::PARTIAL_FLOATS;
    if (is_epi && acc_ok) {
      float* mine = tile_scratch + (size_t)rank * C::PARTIAL_FLOATS;
      for (int c0 = 32 * half; c0 < umma_n; c0 += 64) {
        uint32_t v[32];
#pragma unroll
        for (int a = 0; a < ACCS; ++a) {
          tmem_ld32(t_lane + a * BN + c0, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (c0 + j < n_cols) __stcg(mine + (a * BN + c0 + j) * 128 + fl, __uint_as_float(v[j]));
        }
      }
    }
    __syncwarp();
    if (threadIdx.x == 64) GEMM_TRACE(7);
    KTRACE_T(14, 64);
    cluster_sync_all();   // release/acquire at cluster scope: every partial tile of the cluster is visible
    if (threadIdx.x == 64) GEMM_TRACE(8);
    KTRACE_T(15, 64);
    if (is_epi) {
      // this CTA owns columns rank, rank+split, ...; the two warps of a quarter alternate groups of G of them
      // (all partial-tile loads of a group are in flight together, then the residual loads, then the stores: the loop is
      // a chain of L2 round trips, so a group of 8 columns halves its length against 4)
      constexpr int G = 8;
      const int n_owned = n_cols > rank ? (n_cols - rank + split - 1) / split : 0;
      for (int i0 = G * half; i0 < n_owned; i0 += 2 * G) {
        float s1[G], s2[G];
#pragma unroll
        for (int ci = 0; ci < G; ++ci) {
          const int c = rank + (i0 + ci) * split;
          float a[8], b[8];
#pragma unroll
          for (int r = 0; r < 8; ++r) {
            a[r] = 0.f;
            b[r] = 0.f;
            if (r < split && i0 + ci < n_owned) {
              a[r] = __ldcg(tile_scratch + (size_t)r * C::PARTIAL_FLOATS + c * 128 + fl);
              if (TWO) b[r] = __ldcg(tile_scratch + (size_t)r * C::PARTIAL_FLOATS + (BN + c) * 128 + fl);
            }
          }
          s1[ci] = ((a[0] + a[1]) + (a[2] + a[3])) + ((a[4] + a[5]) + (a[6] + a[7]));
          s2[ci] = ((b[0] + b[1]) + (b[2] + b[3])) + ((b[4] + b[5]) + (b[6] + b[7]));
          if (scaled) {
            const float f = row_scale[min(c, BN - 1)];
            s1[ci] *= f;
            s2[ci] *= f;
          }
        }
        const int n_valid = min(G, n_owned - i0);
        if (m256) {
          gemm_epilogue_cols<G>(p.epi, th_first, tok0 + rank + i0 * split, split, n_valid, s1, s1);
          gemm_epilogue_cols<G>(p.epi, th2, tok0 + rank + i0 * split, split, n_valid, s2, s2);
        } else {
          gemm_epilogue_cols<G>(p.epi, th_first, tok0 + rank + i0 * split, split, n_valid, s1, s2);
        }
      }
    }
    if (threadIdx.x == 64) GEMM_TRACE(9);
    KTRACE_T(16, 64);
  }

  // ---------------- teardown ----------------
  if (threadIdx.x == 64) GEMM_TRACE(11);
  tc_fence_before();
  if (CG2) cluster_sync_all();   // neither CTA of a pair retires while the other may still signal its barriers
  __syncthreads();
  if (threadIdx.x == 0) GEMM_TRACE(12);
  if (*abort_flag) {
    if (threadIdx.x == 0 && p.status) atomicOr(p.status, VLA_ST_WAIT_TIMEOUT);
    for (int i = 0; i < 32; ++i) __nanosleep(1000);   // let any copy still in flight land before the CTA exits
  }
  if (warp == 1) tmem_dealloc(tmem_base, C::TMEM_COLS);
  KTRACE(12);
  if (threadIdx.x == 32) GEMM_TRACE(13);
}
