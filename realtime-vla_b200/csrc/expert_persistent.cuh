// Persistent action-expert kernel: the whole 10-step Euler loop of the 300M expert (single observation) as ONE
// cooperative launch of one CTA per SM, replacing ~930 per-operator launches.
//
// Decomposition (reference loop: pi0_infer.py:1165-1230, pi05_infer.py:418-523):
//   * every GEMM is partitioned over OUTPUT FEATURES with the full K per CTA (8-feature tiles, the n8 of
//     mma.sync.m16n8k16): no split-K exchange, no cluster.  The 51 suffix tokens are the M dimension (4 m16 tiles).
//   * each CTA's weights are pre-packed at load time into ONE contiguous stream of 16 KB chunks (8 features x 1024 K in
//     mma B-fragment order) in exactly the order the CTA consumes them; warp 8 copies the stream into a ring of shared
//     memory slots with cp.async.bulk, decoupled from the phase structure: while the CTA waits at a grid barrier the
//     weights of the next operators keep arriving from HBM.
//   * activations are small (<= 51 x 4096 bf16) and live in L2; a phase reads them with cp.async.cg into swizzled
//     shared memory and feeds the tensor cores with ldmatrix.
//   * phases are separated by grid barriers (one global counter, red.release / ld.acquire, ~1.1 us for 148 CTAs);
//     every spin is bounded by %globaltimer and raises the status word instead of hanging.
//   * the fp32 residual stream is owned by feature: CTA c < 128 keeps x[:, 8c..8c+7] in its shared memory for the whole
//     kernel; what other CTAs read is the bf16 mirror (GEMM operand) and per-CTA partial sums of squares (the RMS
//     norms are folded into the consuming GEMMs: norm(x) @ W = f * (x @ W), pi0_infer.py:1005; Pi05 adaRMS as
//     f * ((x * (1 + scale)) @ W) + shift @ W, pi05_infer.py:78-113).
//   * suffix attention (408 query rows x <= 1024 keys, head dim 256): 32-row blocks x key splits over the CTAs,
//     single-pass softmax per split, partial outputs merged in a second short phase.
#pragma once
#include "common.cuh"

namespace xp {

constexpr int THREADS = 288;          // 8 MMA warps + 1 weight-stream warp
constexpr int CTHREADS = 256;
constexpr int CHUNK_BYTES = 16384;    // 8 features x 1024 K, bf16, fragment order
constexpr int NSLOT = 6;
constexpr int MAX_ROWS = 52;          // suffix tokens held in shared memory
constexpr int A_BYTES = MAX_ROWS * 2048;          // resident A [rows][1024] / 4 streamed stages / K+V of attention
constexpr int STAGE_BYTES = MAX_ROWS * 512;       // streamed A stage: [rows][256 K]
constexpr int SCR_BYTES = 16384;                  // GEMM: K-half exchange (8 KB); attention: Q tile (16 KB)
constexpr int RING_OFF = A_BYTES + SCR_BYTES;
constexpr int PERSIST_OFF = RING_OFF + NSLOT * CHUNK_BYTES;
constexpr int PERSIST_BYTES = 4096;
constexpr int SMEM_BYTES = PERSIST_OFF + PERSIST_BYTES + 128;
constexpr int N_OWNERS = 128;         // CTAs that own 8 features of the 1024-wide stream / 32 hidden features
constexpr int CH_PER_LAYER = 17;      // stream slots per layer: qkv 0-2, o 3-4, (gate,up) x4 5-12, down 13-16
constexpr int ATT_ROWS = 32;          // query rows per attention work item
constexpr int ATT_MAX_KEYS = 96;      // keys per split

struct Params {
  int pi05, S, C, P, T, nl, nsteps, G;
  int att_nrb, att_ks, att_kps;   // row blocks, key splits, keys per split (multiple of 16, <= ATT_MAX_KEYS)
  const uint4* wstream;           // [G][chunks_per_cta][1024] uint4
  int chunks_per_cta;             // nl_alloc * CH_PER_LAYER + 2   (misc: +0 action MLP (Pi0), +1 out projection)
  int misc_base;
  const bf16* w_in;               // action in-projection, K-major [1024][64]
  const float* b_in;              // Pi0: time biases [steps][ld_b_in]; Pi05: bias [1024]
  int ld_b_in;
  const float* b_mlp;             // Pi0 action MLP bias
  const bf16* w_state;            // Pi0 state in-projection, K-major [1024][64]
  const float* b_state;
  const bf16* state;              // [32]
  const float* b_out;             // [32]
  const float* sw_fin;            // Pi05: shift_fin @ W_out per step [steps][32]
  const float *style_attn, *style_ffn, *style_fin;   // Pi05 [step][layer][3072] / [step][3072]
  const float *sw_qkv, *sw_gate, *sw_up;             // Pi05 shift @ W per (step, layer)
  bf16* noise; float* noise_f32; bf16* act; float* x_out; bf16* xb; float* ssq;
  bf16* q; bf16* kcache; bf16* vcache; bf16* attn; bf16* hidden;
  float* att_part; float* att_stat;
  const float *rope_cos, *rope_sin;
  const int *valid_len_ptr, *pos_base_ptr;
  unsigned int* bar_ctr;          // [0] grid-barrier counter, [1] abort word; both zeroed by the host before every launch
  int* status;
  unsigned long long* trace;      // optional timeline of CTA 0: [2 * phase] = arrival, [2 * phase + 1] = release
};

// ---- small PTX wrappers ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// 16-byte global -> shared copy through L2 only; src_bytes = 0 zero-fills the destination
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void cbar() { asm volatile("bar.sync 1, 256;" ::: "memory"); }   // the 8 MMA warps
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar, uint64_t policy) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy) : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
// byte offset of 16-byte chunk `ch` of row `row` in a swizzled tile with `pitch` bytes per row (pitch % 128 == 0)
__host__ __device__ __forceinline__ uint32_t swz(int row, int ch, int pitch) { return (uint32_t)(row * pitch + ((ch ^ (row & 7)) << 4)); }

// ---- shared state ------------------------------------------------------------------------------------------------------
struct Ctx {
  const Params* p;
  uint32_t sbase;         // shared address of the A region
  uint8_t* sptr;          // generic pointer to the same
  uint32_t full_bar, empty_bar;
  volatile int* s_abort;
  float* fs;              // [64] per-token RMS scale
  float* xs;              // [64][8] this CTA's slice of the residual stream
  float* sttok;           // [8]
  unsigned int chunk_g;   // chunks consumed so far (consumer side)
  unsigned int bar_epoch; // grid barriers passed
  int cta, warp, lane, tid;
  int valid_len, pos_base;
  bool fine;
};

// development timeline inside phases: CTA 0, thread 0, Euler step 0, layer 1 only -> trace[2560 + id]
#ifdef XP_FINE_TRACE
#define XP_MARK(c, id) do { if ((c).fine && (c).tid == 0) (c).p->trace[2560 + (id)] = globaltimer_ns(); } while (0)
#else
#define XP_MARK(c, id) do {} while (0)
#endif
__device__ __forceinline__ bool poll_abort(Ctx& c) {
  if (*c.s_abort) return true;
  if (*reinterpret_cast<volatile unsigned int*>(c.p->bar_ctr + 1)) { *c.s_abort = 1; return true; }
  return false;
}
// a bounded wait ran out: tell this CTA, every other CTA (abort word) and the host (sticky status word)
__device__ __forceinline__ void raise_timeout(Ctx& c) {
  *c.s_abort = 1;
  atomicOr(c.p->bar_ctr + 1, 1u);
  atomicOr(c.p->status, VLA_ST_WAIT_TIMEOUT);
}
// bounded mbarrier wait; false = gave up (status word raised) or another CTA / role gave up
__device__ __forceinline__ bool wait_bar(Ctx& c, uint32_t bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  for (;;) {
    for (int i = 0; i < 128; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (poll_abort(c)) return false;
    if (globaltimer_ns() - t0 > VLA_WAIT_LIMIT_NS) {
      raise_timeout(c);
      return false;
    }
  }
}
// shared address of ring slot holding the g-th chunk, after waiting for it
__device__ __forceinline__ uint32_t acquire_chunk(Ctx& c, unsigned int g, bool* ok) {
  const unsigned int s = g % NSLOT;
  if (!wait_bar(c, c.full_bar + 8 * s, (g / NSLOT) & 1u)) *ok = false;
  return c.sbase + RING_OFF + s * CHUNK_BYTES;
}
__device__ __forceinline__ void release_chunk(Ctx& c, unsigned int g) {
  __syncwarp();
  if (c.lane == 0) mbar_arrive(c.empty_bar + 8 * (g % NSLOT));
}

// Grid-wide barrier of the MMA warps of all CTAs.  Returns false after a timeout / abort.
__device__ __forceinline__ bool grid_barrier(Ctx& c, int trace_slot) {
  cbar();
  if (c.tid == 0) {
    const Params& p = *c.p;
    if (p.trace && c.cta == 0) p.trace[2 * trace_slot] = globaltimer_ns();
    ++c.bar_epoch;
    __threadfence();
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.bar_ctr) : "memory");
    const unsigned int target = c.bar_epoch * (unsigned int)p.G;
    const uint64_t t0 = globaltimer_ns();
    unsigned int v, spins = 0;
    for (;;) {
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p.bar_ctr) : "memory");
      if (v >= target) break;
      if ((++spins & 255u) == 0) {
        if (poll_abort(c)) break;
        if (globaltimer_ns() - t0 > VLA_WAIT_LIMIT_NS) {
          raise_timeout(c);
          break;
        }
      }
    }
    __threadfence();
    if (p.trace && c.cta == 0) p.trace[2 * trace_slot + 1] = globaltimer_ns();
  } else {
    ++c.bar_epoch;
  }
  cbar();
  return *c.s_abort == 0;
}

// ---- A operand loaders ---------------------------------------------------------------------------------------------------
// resident: rows x K bf16 (K <= 1024, K % 8 == 0) from global (row pitch ld elements) into the swizzled [rows][2048 B] tile
__device__ __forceinline__ void load_a_resident(Ctx& c, const bf16* src, int rows, int K, int ld) {
  const int cpr = K >> 3;
  for (int idx = c.tid; idx < rows * cpr; idx += CTHREADS) {
    const int row = idx / cpr, ch = idx - row * cpr;
    cp_async16(c.sbase + swz(row, ch, 2048), src + (size_t)row * ld + ch * 8, 16);
  }
  cp_async_commit();
}
// per-token RMS scale from the producers' partial sums of squares: fs[t] = rsqrt(sum_slots ssq[slot][t] / 1024 + 1e-6)
__device__ __forceinline__ void compute_fs(Ctx& c) {
  const int t = c.tid >> 2, part = c.tid & 3;
  float acc = 0.f;
  for (int s = part * 32; s < part * 32 + 32; ++s) acc += __ldcg(c.p->ssq + s * 64 + t);
  acc += __shfl_xor_sync(0xffffffffu, acc, 1);
  acc += __shfl_xor_sync(0xffffffffu, acc, 2);
  if (part == 0) c.fs[t] = rsqrtf(acc * (1.0f / 1024.0f) + 1e-6f);
}

// ---- GEMM cores ------------------------------------------------------------------------------------------------------------
// NT feature tiles (their chunks at slot addresses sl[0..NT-1]) against the resident A tile; this warp's K half.
template <int NT>
__device__ __forceinline__ void mma_resident(const Ctx& c, const uint32_t* sl, int rows, int k_steps_pairs, float (&acc)[NT][4]) {
  const int mi = c.warp & 3, kh = c.warp >> 2;
  float acc2[NT][4];
#pragma unroll
  for (int t = 0; t < NT; ++t)
#pragma unroll
    for (int j = 0; j < 4; ++j) { acc[t][j] = 0.f; acc2[t][j] = 0.f; }
  if (16 * mi >= rows) return;
  const int row = min(16 * mi + (c.lane & 15), rows - 1);
  const uint32_t a_row = c.sbase + row * 2048;
  const int rx = row & 7, hi = c.lane >> 4;
  const int half = k_steps_pairs >> 1;
  const int sp0 = kh * half, sp1 = sp0 + half;
#pragma unroll 4
  for (int sp = sp0; sp < sp1; ++sp) {
    uint4 b[NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) b[t] = lds128(sl[t] + (uint32_t)(sp * 32 + c.lane) * 16);
    uint32_t a0, a1, a2, a3, e0, e1, e2, e3;
    const int kc = 4 * sp + hi;
    ldsm_x4(a_row + (uint32_t)(((kc) ^ rx) << 4), a0, a1, a2, a3);
    ldsm_x4(a_row + (uint32_t)(((kc + 2) ^ rx) << 4), e0, e1, e2, e3);
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      mma16816(acc[t], a0, a1, a2, a3, b[t].x, b[t].y);
      mma16816(acc2[t], e0, e1, e2, e3, b[t].z, b[t].w);
    }
  }
#pragma unroll
  for (int t = 0; t < NT; ++t)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[t][j] += acc2[t][j];
}

// Adds the partial accumulators of the K-half-1 warps to those of the K-half-0 warps through shared memory.  After the
// call the warps with kh == 0 hold the sums.  `buf` alternates between consecutive calls (see the WAR note in the text).
template <int NT>
__device__ __forceinline__ void reduce_khalves(const Ctx& c, int buf, float (&acc)[NT][4]) {
  const int mi = c.warp & 3, kh = c.warp >> 2;
  float4* red = reinterpret_cast<float4*>(c.sptr + A_BYTES) + (size_t)buf * 256;   // [buf][mi][t(2)][lane]
  if (kh == 1) {
#pragma unroll
    for (int t = 0; t < NT; ++t) red[(mi * 2 + t) * 32 + c.lane] = make_float4(acc[t][0], acc[t][1], acc[t][2], acc[t][3]);
  }
  cbar();
  if (kh == 0) {
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      const float4 v = red[(mi * 2 + t) * 32 + c.lane];
      acc[t][0] += v.x; acc[t][1] += v.y; acc[t][2] += v.z; acc[t][3] += v.w;
    }
  }
}

// One feature tile (chunks g0 .. g0 + K/1024 - 1) against A rows streamed from global [rows][K] in 256-wide K stages.
__device__ __forceinline__ bool mma_streamed(Ctx& c, const bf16* src, int rows, int K, float (&acc)[1][4]) {
  const int mi = c.warp & 3, kh = c.warp >> 2;
  const int n_stages = K >> 8;
  bool ok = true;
  float acc2[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int j = 0; j < 4; ++j) acc[0][j] = 0.f;
  auto load_stage = [&](int st) {
    const uint32_t base = c.sbase + (uint32_t)(st & 3) * STAGE_BYTES;
    const bf16* s0 = src + (size_t)st * 256;
    for (int idx = c.tid; idx < rows * 32; idx += CTHREADS) {
      const int row = idx >> 5, ch = idx & 31;
      cp_async16(base + swz(row, ch, 512), s0 + (size_t)row * K + ch * 8, 16);
    }
  };
  XP_MARK(c, K == 2048 ? 20 : 40);
  for (int st = 0; st < 3; ++st) {
    if (st < n_stages) load_stage(st);
    cp_async_commit();
  }
  XP_MARK(c, K == 2048 ? 21 : 41);
  const bool active = 16 * mi < rows;
  const int row = min(16 * mi + (c.lane & 15), rows - 1);
  const int rx = row & 7, hi = c.lane >> 4;
  uint32_t slot = 0;
  for (int st = 0; st < n_stages; ++st) {
    cp_async_wait<2>();
    cbar();
    if (st + 3 < n_stages) load_stage(st + 3);
    cp_async_commit();
    if ((st & 3) == 0) slot = acquire_chunk(c, c.chunk_g + (st >> 2), &ok);
    if (active && ok) {
      const uint32_t a_row = c.sbase + (uint32_t)(st & 3) * STAGE_BYTES + row * 512;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int spl = 4 * kh + i;
        const uint4 b = lds128(slot + (uint32_t)((((st & 3) * 8 + spl) * 32) + c.lane) * 16);
        uint32_t a0, a1, a2, a3, e0, e1, e2, e3;
        const int kc = 4 * spl + hi;
        ldsm_x4(a_row + (uint32_t)((kc ^ rx) << 4), a0, a1, a2, a3);
        ldsm_x4(a_row + (uint32_t)(((kc + 2) ^ rx) << 4), e0, e1, e2, e3);
        mma16816(acc[0], a0, a1, a2, a3, b.x, b.y);
        mma16816(acc2, e0, e1, e2, e3, b.z, b.w);
      }
    }
    if ((st & 3) == 3) release_chunk(c, c.chunk_g + (st >> 2));
    XP_MARK(c, (K == 2048 ? 22 : 42) + st);
  }
  cp_async_wait<0>();
  c.chunk_g += (unsigned int)(K >> 10);
#pragma unroll
  for (int j = 0; j < 4; ++j) acc[0][j] += acc2[j];
  return ok;
}

// ---- epilogues (executed by the four warps with kh == 0; thread holds rows r0 = 16 mi + lane/4 and r0 + 8, features n, n+1) --
struct ResidEpi {
  int rows;          // valid A rows
  int row_off;       // output token = A row + row_off
  bool accumulate;   // x += gate * acc (else x = acc + bias)
  const float* bias; // [1024] or null
  const float* gate; // [1024] or null (1)
  const float* mscale;  // [1024] or null: mirror = x * (1 + mscale[n])
};
// residual-stream update for this CTA's 8 features; writes the bf16 mirror, the fp32 copy and the partial sums of squares
__device__ __forceinline__ void epi_resid(Ctx& c, const ResidEpi& e, const float* acc) {
  const Params& p = *c.p;
  const int mi = c.warp & 3;
  const int j0 = 2 * (c.lane & 3), n = 8 * c.cta + j0;
  const float b0 = e.bias ? e.bias[n] : 0.f, b1 = e.bias ? e.bias[n + 1] : 0.f;
  const float g0 = e.gate ? e.gate[n] : 1.f, g1 = e.gate ? e.gate[n + 1] : 1.f;
  const float m0 = e.mscale ? 1.f + e.mscale[n] : 1.f, m1 = e.mscale ? 1.f + e.mscale[n + 1] : 1.f;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = 16 * mi + (c.lane >> 2) + 8 * h;
    const bool valid = r < e.rows;
    const int t = r + e.row_off;
    float v0 = 0.f, v1 = 0.f;
    if (valid) {
      if (e.accumulate) {
        v0 = c.xs[t * 8 + j0] + g0 * acc[2 * h];
        v1 = c.xs[t * 8 + j0 + 1] + g1 * acc[2 * h + 1];
      } else {
        v0 = acc[2 * h] + b0;
        v1 = acc[2 * h + 1] + b1;
      }
      c.xs[t * 8 + j0] = v0;
      c.xs[t * 8 + j0 + 1] = v1;
      *reinterpret_cast<uint32_t*>(p.xb + (size_t)t * 1024 + n) = pack_bf16x2(v0 * m0, v1 * m1);
      *reinterpret_cast<float2*>(p.x_out + (size_t)t * 1024 + n) = make_float2(v0, v1);
    }
    float sq = v0 * v0 + v1 * v1;
    sq += __shfl_xor_sync(0xffffffffu, sq, 1);
    sq += __shfl_xor_sync(0xffffffffu, sq, 2);
    if (valid && (c.lane & 3) == 0) p.ssq[c.cta * 64 + t] = sq;
  }
}

// ---- phases ----------------------------------------------------------------------------------------------------------------
// Action in-projection (K = 32) straight from global weights: Pi0 -> act = silu(noise @ W + time_bias[step]);
// Pi05 -> x = noise @ W + b (start of the residual stream).  CTA c < 128 owns features 8c..8c+7.
__device__ __forceinline__ void phase_in_proj(Ctx& c, int step) {
  const Params& p = *c.p;
  if (c.cta >= N_OWNERS) return;
  load_a_resident(c, p.noise, p.C, 32, 32);
  cp_async_wait<0>();
  cbar();
  const int mi = c.warp & 3, kh = c.warp >> 2;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  if (kh == 0 && 16 * mi < p.C) {
    const int row = min(16 * mi + (c.lane & 15), p.C - 1);
    const uint32_t a_row = c.sbase + row * 2048;
    const int rx = row & 7, hi = c.lane >> 4;
    const int nb = 8 * c.cta + (c.lane >> 2);
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      uint32_t a0, a1, a2, a3;
      ldsm_x4(a_row + (uint32_t)(((2 * s + hi) ^ rx) << 4), a0, a1, a2, a3);
      const bf16* w = p.w_in + (size_t)nb * 64 + 16 * s + 2 * (c.lane & 3);
      const uint32_t b0 = *reinterpret_cast<const uint32_t*>(w), b1 = *reinterpret_cast<const uint32_t*>(w + 8);
      mma16816(acc, a0, a1, a2, a3, b0, b1);
    }
  }
  if (kh == 0) {
    if (!p.pi05) {
      const int j0 = 2 * (c.lane & 3), n = 8 * c.cta + j0;
      const float* tb = p.b_in + (size_t)step * p.ld_b_in;
      const float b0 = tb[n], b1 = tb[n + 1];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int r = 16 * mi + (c.lane >> 2) + 8 * h;
        if (r < p.C)
          *reinterpret_cast<uint32_t*>(p.act + (size_t)r * 1024 + n) = pack_bf16x2(silu_f(acc[2 * h] + b0), silu_f(acc[2 * h + 1] + b1));
      }
    } else {
      ResidEpi e;
      e.rows = p.C; e.row_off = 0; e.accumulate = false; e.bias = p.b_in; e.gate = nullptr;
      e.mscale = p.style_attn + (size_t)step * p.nl * 3072;   // pre-attention norm of layer 0
      epi_resid(c, e, acc);
    }
  }
}

// Pi0 action MLP: x[1 + a] = act[a] @ W + b; x[0] = state token.
__device__ __forceinline__ bool phase_action_mlp(Ctx& c) {
  const Params& p = *c.p;
  if (c.cta >= N_OWNERS) return true;
  bool ok = true;
  load_a_resident(c, p.act, p.C, 1024, 1024);
  const uint32_t sl = acquire_chunk(c, c.chunk_g, &ok);
  cp_async_wait<0>();
  cbar();
  float acc[1][4];
  if (ok) mma_resident<1>(c, &sl, p.C, 32, acc);
  release_chunk(c, c.chunk_g);
  c.chunk_g += 1;
  reduce_khalves<1>(c, 0, acc);
  if ((c.warp >> 2) == 0) {
    ResidEpi e;
    e.rows = p.C; e.row_off = 1; e.accumulate = false; e.bias = p.b_mlp; e.gate = nullptr; e.mscale = nullptr;
    epi_resid(c, e, acc[0]);
  }
  if (c.tid < 8) {   // the state token row (constant over the Euler steps)
    const float v = c.sttok[c.tid];
    c.xs[c.tid] = v;
    p.xb[8 * c.cta + c.tid] = __float2bfloat16(v);
    p.x_out[8 * c.cta + c.tid] = v;
    float sq = v * v;
    sq += __shfl_xor_sync(0xffu, sq, 1);
    sq += __shfl_xor_sync(0xffu, sq, 2);
    sq += __shfl_xor_sync(0xffu, sq, 4);
    if (c.tid == 0) p.ssq[c.cta * 64] = sq;
  }
  return ok;
}

// QKV projection with folded norm, rotary embedding and K/V-cache append (pi0_infer.py:777-810).
// CTA c owns feature tiles c, c + G, c + 2G (< 320).
__device__ __forceinline__ bool phase_qkv(Ctx& c, int step, int layer) {
  const Params& p = *c.p;
  bool ok = true;
  const int nq = (c.cta + 2 * p.G < 320) ? 3 : ((c.cta + p.G < 320) ? 2 : (c.cta < 320 ? 1 : 0));
  if (nq == 0) return true;
  XP_MARK(c, 0);
  load_a_resident(c, p.xb, p.S, 1024, 1024);
  XP_MARK(c, 1);
  compute_fs(c);
  XP_MARK(c, 2);
  uint32_t sl[3];
  for (int j = 0; j < nq; ++j) sl[j] = acquire_chunk(c, c.chunk_g + j, &ok);
  XP_MARK(c, 3);
  cp_async_wait<0>();
  XP_MARK(c, 4);
  cbar();
  XP_MARK(c, 5);
  const int mi = c.warp & 3, kh = c.warp >> 2;
  const float* bias = p.pi05 ? p.sw_qkv + ((size_t)step * p.nl + layer) * 2560 : nullptr;
  bf16* kc = p.kcache + (size_t)layer * p.T * 256;
  bf16* vc = p.vcache + (size_t)layer * p.T * 256;
  auto epilogue = [&](int tile, const float* acc) {
    const int n = 8 * tile + 2 * (c.lane & 3);
    const float b0 = bias ? bias[n] : 0.f, b1 = bias ? bias[n + 1] : 0.f;
    const bool rot = n < 2304;
    const int fi = (n & 255) >> 1;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = 16 * mi + (c.lane >> 2) + 8 * h;
      if (r >= p.S) continue;
      const float f = c.fs[r];
      float v0 = f * acc[2 * h] + b0, v1 = f * acc[2 * h + 1] + b1;
      if (rot) {
        const int pos = c.pos_base + r;
        const float cs = p.rope_cos[pos * 128 + fi], sn = p.rope_sin[pos * 128 + fi];
        const float y0 = v0 * cs - v1 * sn, y1 = v1 * cs + v0 * sn;
        v0 = y0; v1 = y1;
      }
      const uint32_t o = pack_bf16x2(v0, v1);
      if (n < 2048) *reinterpret_cast<uint32_t*>(p.q + (size_t)r * 2048 + n) = o;
      else if (n < 2304) *reinterpret_cast<uint32_t*>(kc + (size_t)(p.P + r) * 256 + (n - 2048)) = o;
      else *reinterpret_cast<uint32_t*>(vc + (size_t)(p.P + r) * 256 + (n - 2304)) = o;
    }
  };
  {
    float acc[2][4];
    if (nq >= 2) {
      if (ok) mma_resident<2>(c, sl, p.S, 32, acc);
      XP_MARK(c, 6);
      release_chunk(c, c.chunk_g);
      release_chunk(c, c.chunk_g + 1);
      reduce_khalves<2>(c, 0, acc);
      XP_MARK(c, 7);
      if (kh == 0) { epilogue(c.cta, acc[0]); epilogue(c.cta + p.G, acc[1]); }
      XP_MARK(c, 8);
    }
    if (nq == 1 || nq == 3) {
      float a1[1][4];
      const uint32_t s1 = sl[nq - 1];
      if (ok) mma_resident<1>(c, &s1, p.S, 32, a1);
      release_chunk(c, c.chunk_g + nq - 1);
      reduce_khalves<1>(c, 1, a1);
      if (kh == 0) epilogue(c.cta + (nq - 1) * p.G, a1[0]);
      XP_MARK(c, 9);
    }
  }
  c.chunk_g += (unsigned int)nq;
  return ok;
}

// GeGLU: hidden[:, 32c..32c+31] = gelu(f * (xb @ Wg) + bg) * (f * (xb @ Wu) + bu), four (gate, up) tile pairs per CTA.
__device__ __forceinline__ bool phase_geglu(Ctx& c, int step, int layer) {
  const Params& p = *c.p;
  if (c.cta >= N_OWNERS) return true;
  bool ok = true;
  XP_MARK(c, 60);
  load_a_resident(c, p.xb, p.S, 1024, 1024);
  compute_fs(c);
  cp_async_wait<0>();
  cbar();
  XP_MARK(c, 61);
  const int mi = c.warp & 3, kh = c.warp >> 2;
  const float* bg = p.pi05 ? p.sw_gate + ((size_t)step * p.nl + layer) * 4096 : nullptr;
  const float* bu = p.pi05 ? p.sw_up + ((size_t)step * p.nl + layer) * 4096 : nullptr;
  for (int i = 0; i < 4; ++i) {
    uint32_t sl[2];
    sl[0] = acquire_chunk(c, c.chunk_g, &ok);
    sl[1] = acquire_chunk(c, c.chunk_g + 1, &ok);
    XP_MARK(c, 62 + 4 * i);
    float acc[2][4];
    if (ok) mma_resident<2>(c, sl, p.S, 32, acc);
    XP_MARK(c, 63 + 4 * i);
    release_chunk(c, c.chunk_g);
    release_chunk(c, c.chunk_g + 1);
    c.chunk_g += 2;
    reduce_khalves<2>(c, i & 1, acc);
    XP_MARK(c, 64 + 4 * i);
    if (kh == 0) {
      const int n = 32 * c.cta + 8 * i + 2 * (c.lane & 3);
      const float g0 = bg ? bg[n] : 0.f, g1 = bg ? bg[n + 1] : 0.f, u0 = bu ? bu[n] : 0.f, u1 = bu ? bu[n + 1] : 0.f;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int r = 16 * mi + (c.lane >> 2) + 8 * h;
        if (r >= p.S) continue;
        const float f = c.fs[r];
        const float h0 = gelu_tanh_f(f * acc[0][2 * h] + g0) * (f * acc[1][2 * h] + u0);
        const float h1 = gelu_tanh_f(f * acc[0][2 * h + 1] + g1) * (f * acc[1][2 * h + 1] + u1);
        *reinterpret_cast<uint32_t*>(p.hidden + (size_t)r * 4096 + n) = pack_bf16x2(h0, h1);
      }
    }
    XP_MARK(c, 65 + 4 * i);
  }
  return ok;
}

// Attention-out (K = 2048) and MLP-down (K = 4096) projections with the residual add.
__device__ __forceinline__ bool phase_resid(Ctx& c, const bf16* a_src, int K, const float* gate, const float* mscale) {
  const Params& p = *c.p;
  if (c.cta >= N_OWNERS) return true;
  float acc[1][4];
  const bool ok = mma_streamed(c, a_src, p.S, K, acc);
  reduce_khalves<1>(c, 0, acc);
  XP_MARK(c, K == 2048 ? 38 : 58);
  if ((c.warp >> 2) == 0) {
    ResidEpi e;
    e.rows = p.S; e.row_off = 0; e.accumulate = true; e.bias = nullptr; e.gate = gate; e.mscale = mscale;
    epi_resid(c, e, acc[0]);
  }
  XP_MARK(c, K == 2048 ? 39 : 59);
  return ok;
}

// Out projection + Euler update: noise += f * (xb[action rows] @ W_out) + b  (pi0_infer.py:1224-1230).  CTA c < 4.
__device__ __forceinline__ bool phase_out(Ctx& c, int step) {
  const Params& p = *c.p;
  if (c.cta >= 4) return true;
  bool ok = true;
  const int off = p.pi05 ? 0 : 1;
  load_a_resident(c, p.xb + (size_t)off * 1024, p.C, 1024, 1024);
  compute_fs(c);
  const uint32_t sl = acquire_chunk(c, c.chunk_g, &ok);
  cp_async_wait<0>();
  cbar();
  float acc[1][4];
  if (ok) mma_resident<1>(c, &sl, p.C, 32, acc);
  release_chunk(c, c.chunk_g);
  c.chunk_g += 1;
  reduce_khalves<1>(c, 0, acc);
  if ((c.warp >> 2) == 0) {
    const int mi = c.warp & 3;
    const int n = 8 * c.cta + 2 * (c.lane & 3);
    float b0 = p.b_out[n], b1 = p.b_out[n + 1];
    if (p.pi05) { b0 += p.sw_fin[step * 32 + n]; b1 += p.sw_fin[step * 32 + n + 1]; }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = 16 * mi + (c.lane >> 2) + 8 * h;
      if (r >= p.C) continue;
      const float f = c.fs[r + off];
      float o0, o1;
      if (step == 0) {
        const __nv_bfloat162 nz = *reinterpret_cast<const __nv_bfloat162*>(p.noise + (size_t)r * 32 + n);
        o0 = __low2float(nz); o1 = __high2float(nz);
      } else {
        const float2 nz = __ldcg(reinterpret_cast<const float2*>(p.noise_f32 + (size_t)r * 32 + n));
        o0 = nz.x; o1 = nz.y;
      }
      o0 += f * acc[0][2 * h] + b0;
      o1 += f * acc[0][2 * h + 1] + b1;
      *reinterpret_cast<float2*>(p.noise_f32 + (size_t)r * 32 + n) = make_float2(o0, o1);
      *reinterpret_cast<uint32_t*>(p.noise + (size_t)r * 32 + n) = pack_bf16x2(o0, o1);
    }
  }
  return ok;
}

// Suffix attention, part 1: work item (row block rb, key split sp) = 32 query rows (4 tokens x 8 heads) against
// <= 96 keys; softmax within the split; unnormalised output and (max, sum) go to the merge buffers.
// Visibility (pi0_infer.py:1069-1095, pi05_infer.py:382-416): key j is visible if (j < valid_len or j >= P), and the
// first `restrict` rows (the Pi0 state token's 8 heads) only see keys j <= P.
__device__ __forceinline__ void phase_attention(Ctx& c, int layer) {
  const Params& p = *c.p;
  const int n_items = p.att_nrb * p.att_ks;
  if (c.cta >= n_items) return;
  const int rb = c.cta / p.att_ks, sp = c.cta - rb * p.att_ks;
  const int R = p.S * 8;
  const int r0 = rb * ATT_ROWS;
  const int key0 = sp * p.att_kps;
  const int nk = max(0, min(p.att_kps, p.T - key0));          // real keys of this split
  const int nkp = (nk + 15) & ~15;                            // padded to the mma K step
  const uint32_t sQ = c.sbase + A_BYTES, sK = c.sbase, sV = c.sbase + ATT_MAX_KEYS * 512;
  const uint32_t sP = c.sbase + 2 * ATT_MAX_KEYS * 512;       // bf16 [32][104] (pitch 208 B)
  float* red = reinterpret_cast<float*>(c.sptr + 2 * ATT_MAX_KEYS * 512 + 32 * 208);   // rmax[4][32], rsum[4][32]
  const bf16* kc = p.kcache + ((size_t)layer * p.T + key0) * 256;
  const bf16* vc = p.vcache + ((size_t)layer * p.T + key0) * 256;
  for (int idx = c.tid; idx < ATT_ROWS * 32; idx += CTHREADS) {
    const int row = idx >> 5, ch = idx & 31;
    const bool v = r0 + row < R;
    cp_async16(sQ + swz(row, ch, 512), p.q + (size_t)(v ? r0 + row : 0) * 256 + ch * 8, v ? 16 : 0);
  }
  for (int idx = c.tid; idx < nkp * 32; idx += CTHREADS) {
    const int row = idx >> 5, ch = idx & 31;
    const bool v = row < nk;
    cp_async16(sK + swz(row, ch, 512), kc + (size_t)(v ? row : 0) * 256 + ch * 8, v ? 16 : 0);
    cp_async16(sV + swz(row, ch, 512), vc + (size_t)(v ? row : 0) * 256 + ch * 8, v ? 16 : 0);
  }
  XP_MARK(c, 10);
  cp_async_commit();
  cp_async_wait<0>();
  cbar();
  XP_MARK(c, 11);

  const int mi = c.warp & 1, grp = c.warp >> 1;     // 16-row tile, key group (S) / 64-dim group (O)
  const int restrict_rows = p.pi05 ? 0 : 8;
  const float scale = 0.0625f * 1.4426950408889634f;
  // ---- S = Q K^T for key tiles grp, grp + 4, grp + 8 ----
  float s[3][4];
#pragma unroll
  for (int t = 0; t < 3; ++t)
#pragma unroll
    for (int j = 0; j < 4; ++j) s[t][j] = 0.f;
  const int n_kt = nkp >> 3;
  {
    const int qrow = 16 * mi + (c.lane & 15);
    const uint32_t q_row = sQ + qrow * 512;
    const int qx = qrow & 7, hi = c.lane >> 4;
#pragma unroll 2
    for (int k2 = 0; k2 < 8; ++k2) {      // two k16 steps per iteration (32 dims)
      uint32_t a0, a1, a2, a3, e0, e1, e2, e3;
      ldsm_x4(q_row + (uint32_t)(((4 * k2 + hi) ^ qx) << 4), a0, a1, a2, a3);
      ldsm_x4(q_row + (uint32_t)(((4 * k2 + 2 + hi) ^ qx) << 4), e0, e1, e2, e3);
#pragma unroll
      for (int t = 0; t < 3; ++t) {
        const int kt = grp + 4 * t;
        if (kt < n_kt) {
          const int krow = 8 * kt + (c.lane & 7);
          uint32_t b0, b1, b2, b3;
          ldsm_x4(sK + krow * 512 + (uint32_t)(((4 * k2 + (c.lane >> 3)) ^ (krow & 7)) << 4), b0, b1, b2, b3);
          mma16816(s[t], a0, a1, a2, a3, b0, b1);
          mma16816(s[t], e0, e1, e2, e3, b2, b3);
        }
      }
    }
  }
  XP_MARK(c, 12);
  // ---- mask, row max over the split ----
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int t = 0; t < 3; ++t) {
    const int kt = grp + 4 * t;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int row = r0 + 16 * mi + (c.lane >> 2) + 8 * (j >> 1);
      const int key = key0 + 8 * kt + 2 * (c.lane & 3) + (j & 1);
      bool vis = kt < n_kt && key < p.T && row < R && (key < c.valid_len || key >= p.P);
      if (row < restrict_rows && key > p.P) vis = false;
      s[t][j] = vis ? s[t][j] * scale : -INFINITY;
      mx[j >> 1] = fmaxf(mx[j >> 1], s[t][j]);
    }
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
    if ((c.lane & 3) == 0) red[grp * 32 + 16 * mi + (c.lane >> 2) + 8 * h] = mx[h];
  }
  cbar();
  float m[2], sum[2] = {0.f, 0.f};
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int rl = 16 * mi + (c.lane >> 2) + 8 * h;
    m[h] = fmaxf(fmaxf(red[rl], red[32 + rl]), fmaxf(red[64 + rl], red[96 + rl]));
  }
  // ---- P = exp2(S - m) as bf16 into shared memory, row sums ----
#pragma unroll
  for (int t = 0; t < 3; ++t) {
    const int kt = grp + 4 * t;
    if (kt < n_kt) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const float mm = m[h] == -INFINITY ? 0.f : m[h];
        const float p0 = exp2f(s[t][2 * h] - mm), p1 = exp2f(s[t][2 * h + 1] - mm);
        const uint32_t pk = pack_bf16x2(p0, p1);
        // the sums use the rounded probabilities, the values the PV product sees
        const __nv_bfloat162 pb = *reinterpret_cast<const __nv_bfloat162*>(&pk);
        sum[h] += __low2float(pb) + __high2float(pb);
        const int rl = 16 * mi + (c.lane >> 2) + 8 * h;
        asm volatile("st.shared.b32 [%0], %1;" ::"r"(sP + rl * 208 + (8 * kt + 2 * (c.lane & 3)) * 2), "r"(pk) : "memory");
      }
    }
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 1);
    sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 2);
    if ((c.lane & 3) == 0) red[128 + grp * 32 + 16 * mi + (c.lane >> 2) + 8 * h] = sum[h];
  }
  cbar();
  XP_MARK(c, 13);
  // ---- O = P V for dims 64 grp .. 64 grp + 63 ----
  float o[8][4];
#pragma unroll
  for (int t = 0; t < 8; ++t)
#pragma unroll
    for (int j = 0; j < 4; ++j) o[t][j] = 0.f;
  {
    const int prow = 16 * mi + (c.lane & 15);
    for (int ks = 0; ks < (nkp >> 4); ++ks) {
      uint32_t a0, a1, a2, a3;
      ldsm_x4(sP + prow * 208 + (uint32_t)((2 * ks + (c.lane >> 4)) << 4), a0, a1, a2, a3);
      const int vrow = 16 * ks + (c.lane & 7) + 8 * ((c.lane >> 3) & 1);
#pragma unroll
      for (int t2 = 0; t2 < 4; ++t2) {     // two 8-dim tiles per ldmatrix
        const int ch = 8 * grp + 2 * t2 + (c.lane >> 4);
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(sV + vrow * 512 + (uint32_t)((ch ^ (vrow & 7)) << 4), b0, b1, b2, b3);
        mma16816(o[2 * t2], a0, a1, a2, a3, b0, b1);
        mma16816(o[2 * t2 + 1], a0, a1, a2, a3, b2, b3);
      }
    }
  }
  XP_MARK(c, 14);
  // ---- partial results ----
  float* part = p.att_part + (size_t)c.cta * ATT_ROWS * 256;
#pragma unroll
  for (int t = 0; t < 8; ++t) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int rl = 16 * mi + (c.lane >> 2) + 8 * h;
      __stcg(reinterpret_cast<float2*>(part + rl * 256 + 64 * grp + 8 * t + 2 * (c.lane & 3)), make_float2(o[t][2 * h], o[t][2 * h + 1]));
    }
  }
  if (c.tid < ATT_ROWS) {
    const int rl = c.tid;
    const float mm = fmaxf(fmaxf(red[rl], red[32 + rl]), fmaxf(red[64 + rl], red[96 + rl]));
    const float l = red[128 + rl] + red[160 + rl] + red[192 + rl] + red[224 + rl];
    __stcg(reinterpret_cast<float2*>(p.att_stat + ((size_t)c.cta * ATT_ROWS + rl) * 2), make_float2(mm, l));
  }
  XP_MARK(c, 15);
}

// Suffix attention, part 2: rows are dealt round-robin to the CTAs; thread d merges dimension d over the key splits.
__device__ __forceinline__ void phase_attention_merge(Ctx& c) {
  const Params& p = *c.p;
  const int R = p.S * 8, ks = p.att_ks;
  XP_MARK(c, 16);
  for (int r = c.cta; r < R; r += p.G) {
    const int rb = r / ATT_ROWS, rl = r - rb * ATT_ROWS;
    float mx = -INFINITY;
    for (int s = 0; s < ks; ++s) mx = fmaxf(mx, __ldcg(p.att_stat + ((size_t)(rb * ks + s) * ATT_ROWS + rl) * 2));
    float L = 0.f, acc = 0.f;
    for (int s = 0; s < ks; ++s) {
      const float2 st = __ldcg(reinterpret_cast<const float2*>(p.att_stat + ((size_t)(rb * ks + s) * ATT_ROWS + rl) * 2));
      const float w = st.x == -INFINITY ? 0.f : exp2f(st.x - mx);
      L += w * st.y;
      acc += w * __ldcg(p.att_part + ((size_t)(rb * ks + s) * ATT_ROWS + rl) * 256 + c.tid);
    }
    p.attn[(size_t)r * 256 + c.tid] = __float2bfloat16(acc / L);
  }
  XP_MARK(c, 17);
}

// ---- weight stream (warp 8, one lane) ---------------------------------------------------------------------------------------
__device__ __forceinline__ void producer_loop(Ctx& c) {
  const Params& p = *c.p;
  const uint4* base = p.wstream + (size_t)c.cta * p.chunks_per_cta * (CHUNK_BYTES / 16);
  const uint64_t pol = policy_evict_first();
  unsigned int g = 0;
  bool ok = true;
  auto push = [&](int idx) {
    if (!ok) return;
    const unsigned int s = g % NSLOT;
    if (g >= NSLOT) ok = wait_bar(c, c.empty_bar + 8 * s, ((g / NSLOT) - 1) & 1u);
    if (!ok) return;
    mbar_expect_tx(c.full_bar + 8 * s, CHUNK_BYTES);
    bulk_g2s(c.sbase + RING_OFF + s * CHUNK_BYTES, base + (size_t)idx * (CHUNK_BYTES / 16), CHUNK_BYTES, c.full_bar + 8 * s, pol);
    ++g;
  };
  const int nq = (c.cta + 2 * p.G < 320) ? 3 : ((c.cta + p.G < 320) ? 2 : (c.cta < 320 ? 1 : 0));
  const bool owner = c.cta < N_OWNERS;
  for (int step = 0; step < p.nsteps && ok; ++step) {
    if (!p.pi05 && owner) push(p.misc_base);
    for (int l = 0; l < p.nl && ok; ++l) {
      for (int j = 0; j < nq; ++j) push(l * CH_PER_LAYER + j);
      if (owner)
        for (int j = 3; j < CH_PER_LAYER; ++j) push(l * CH_PER_LAYER + j);
    }
    if (c.cta < 4) push(p.misc_base + 1);
  }
  if (!ok) {
    // give the copies still in flight time to land before the CTA can retire (bounded)
    for (unsigned int i = (g > NSLOT ? g - NSLOT : 0); i < g; ++i) {
      const uint32_t bar = c.full_bar + 8 * (i % NSLOT);
      for (int tries = 0; tries < 20000 && !mbar_try_wait(bar, (i / NSLOT) & 1u); ++tries) __nanosleep(50);
    }
  }
}

// ---- the kernel ----------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(THREADS, 1) expert_persistent_kernel(const __grid_constant__ Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t pad = (128u - (raw & 127u)) & 127u;
  Ctx c;
  c.p = &p;
  c.sbase = raw + pad;
  c.sptr = smem_raw + pad;
  uint8_t* persist = c.sptr + PERSIST_OFF;
  c.full_bar = c.sbase + PERSIST_OFF;
  c.empty_bar = c.full_bar + 8 * NSLOT;
  c.s_abort = reinterpret_cast<volatile int*>(persist + 128);
  c.fs = reinterpret_cast<float*>(persist + 256);
  c.xs = reinterpret_cast<float*>(persist + 512);        // 64 x 8 floats = 2 KB
  c.sttok = reinterpret_cast<float*>(persist + 2560);
  c.chunk_g = 0;
  c.bar_epoch = 0;
  c.fine = false;
  c.cta = blockIdx.x;
  c.tid = threadIdx.x;
  c.warp = threadIdx.x >> 5;
  c.lane = threadIdx.x & 31;
  c.valid_len = p.valid_len_ptr ? *p.valid_len_ptr : p.P;
  c.pos_base = p.pi05 ? (p.pos_base_ptr ? *p.pos_base_ptr : p.P - 1) : p.P;
  if (threadIdx.x == 0) {
    for (int s = 0; s < NSLOT; ++s) {
      mbar_init(c.full_bar + 8 * s, 1);
      mbar_init(c.empty_bar + 8 * s, 8);
    }
    *c.s_abort = 0;
    mbar_fence_init();
  }
  for (int i = threadIdx.x; i < 64 * 8; i += THREADS) c.xs[i] = 0.f;
  __syncthreads();

  if (c.warp == 8) {
    if (c.lane == 0) producer_loop(c);
    __syncwarp();
  } else {
    bool ok = true;
    int ph = 0;   // phase counter (trace slot)
    if (!p.pi05 && c.cta < N_OWNERS && c.tid < 8) {   // state token features of this CTA (pi0_infer.py:1166-1171)
      const int n = 8 * c.cta + c.tid;
      float acc = p.b_state[n];
      for (int k = 0; k < 32; ++k) acc += __bfloat162float(p.state[k]) * __bfloat162float(p.w_state[(size_t)n * 64 + k]);
      c.sttok[c.tid] = acc;
    }
    for (int step = 0; step < p.nsteps && ok; ++step) {
      phase_in_proj(c, step);
      ok = grid_barrier(c, ph++);
      if (!p.pi05 && ok) {
        ok = phase_action_mlp(c);
        ok = grid_barrier(c, ph++) && ok;
      }
      for (int l = 0; l < p.nl && ok; ++l) {
        c.fine = p.trace != nullptr && c.cta == 0 && step == 0 && l == 1;
        ok = phase_qkv(c, step, l);
        ok = grid_barrier(c, ph++) && ok;
        if (!ok) break;
        phase_attention(c, l);
        ok = grid_barrier(c, ph++);
        if (!ok) break;
        phase_attention_merge(c);
        ok = grid_barrier(c, ph++);
        if (!ok) break;
        const size_t sl = (size_t)step * p.nl + l;
        ok = phase_resid(c, p.attn, 2048, p.pi05 ? p.style_attn + sl * 3072 + 2048 : nullptr,
                         p.pi05 ? p.style_ffn + sl * 3072 : nullptr);
        ok = grid_barrier(c, ph++) && ok;
        if (!ok) break;
        ok = phase_geglu(c, step, l);
        ok = grid_barrier(c, ph++) && ok;
        if (!ok) break;
        const float* next_scale = nullptr;
        if (p.pi05) next_scale = (l + 1 < p.nl) ? p.style_attn + (sl + 1) * 3072 : p.style_fin + (size_t)step * 3072;
        ok = phase_resid(c, p.hidden, 4096, p.pi05 ? p.style_ffn + sl * 3072 + 2048 : nullptr, next_scale);
        ok = grid_barrier(c, ph++) && ok;
      }
      if (!ok) break;
      ok = phase_out(c, step);
      ok = grid_barrier(c, ph++) && ok;
    }
    if (!ok) *c.s_abort = 1;
  }
  __syncthreads();
}

// ---- weight packing ----------------------------------------------------------------------------------------------------------
// One 16 KB chunk = features n0..n0+7, K range k0..k0+1023 of a K-major weight w [n_rows][Kp], in the order the MMA
// warps read it: [k-step pair sp (32)][lane (32)][8 bf16] with, for k-step s = 2 sp + (j >> 2) and jj = j & 3,
// element j = W[n0 + lane / 4][k0 + 16 s + 8 (jj >> 1) + 2 (lane % 4) + (jj & 1)]  (the B fragment of mma.m16n8k16).
// Features >= n_valid and K >= k_valid are zero.
__host__ __device__ __forceinline__ void chunk_elem_src(int e, int* n_local, int* k_local) {
  const int j = e & 7, lane = (e >> 3) & 31, sp = e >> 8;
  const int s = 2 * sp + (j >> 2), jj = j & 3;
  *n_local = lane >> 2;
  *k_local = 16 * s + 8 * (jj >> 1) + 2 * (lane & 3) + (jj & 1);
}
__global__ void pack_chunk_kernel(const bf16* __restrict__ w, int Kp, int n_valid, int k_valid, int n0, int k0, bf16* __restrict__ dst) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= CHUNK_BYTES / 2) return;
  int nl, kl;
  chunk_elem_src(e, &nl, &kl);
  const int n = n0 + nl, k = k0 + kl;
  dst[e] = (n < n_valid && k < k_valid) ? w[(size_t)n * Kp + k] : __float2bfloat16(0.f);
}
// All chunks of one expert layer: grid (CH_PER_LAYER, G).  Stream slot j of CTA c holds (K-major sources, layer l):
//   j = 0..2   QKV feature tile c + j G (if < 320), K 0..1023
//   j = 3..4   attention-out tile c, K half j - 3                      (c < N_OWNERS from here on)
//   j = 5..12  MLP gate (odd offsets: up) tile 4 c + (j - 5) / 2
//   j = 13..16 MLP down tile c, K quarter j - 13
__global__ void pack_layer_kernel(const bf16* __restrict__ w_qkv, const bf16* __restrict__ w_o, const bf16* __restrict__ w_gate,
                                  const bf16* __restrict__ w_up, const bf16* __restrict__ w_down, int layer, int chunks_per_cta,
                                  bf16* __restrict__ stream) {
  const int j = blockIdx.x, cta = blockIdx.y, G = gridDim.y;
  const bf16* src;
  int Kp, n0, k0;
  if (j < 3) {
    const int tile = cta + j * G;
    if (tile >= 320) return;
    src = w_qkv; Kp = 1024; n0 = 8 * tile; k0 = 0;
  } else {
    if (cta >= N_OWNERS) return;
    if (j < 5) { src = w_o; Kp = 2048; n0 = 8 * cta; k0 = 1024 * (j - 3); }
    else if (j < 13) { src = ((j - 5) & 1) ? w_up : w_gate; Kp = 1024; n0 = 32 * cta + 8 * ((j - 5) >> 1); k0 = 0; }
    else { src = w_down; Kp = 4096; n0 = 8 * cta; k0 = 1024 * (j - 13); }
  }
  bf16* dst = stream + ((size_t)cta * chunks_per_cta + (size_t)layer * CH_PER_LAYER + j) * (CHUNK_BYTES / 2);
  for (int e = threadIdx.x; e < CHUNK_BYTES / 2; e += blockDim.x) {
    int nl, kl;
    chunk_elem_src(e, &nl, &kl);
    dst[e] = src[(size_t)(n0 + nl) * Kp + k0 + kl];
  }
}

// Pi05: sw_fin[step][n] = sum_k bf16(shift_fin[step][k]) * W_out[n][k]  (shift third of the final adaRMS style row)
__global__ void sw_fin_kernel(const float* __restrict__ style_fin, const bf16* __restrict__ w_out, int Kp, int n_steps, float* __restrict__ out) {
  const int step = blockIdx.x, n = threadIdx.x >> 5, lane = threadIdx.x & 31;   // 32 warps = 32 features
  if (step >= n_steps) return;
  float acc = 0.f;
  for (int k = lane; k < 1024; k += 32)
    acc += __bfloat162float(__float2bfloat16(style_fin[(size_t)step * 3072 + 1024 + k])) * __bfloat162float(w_out[(size_t)n * Kp + k]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) out[step * 32 + n] = acc;
}

}  // namespace xp
