// Persistent action-expert kernel: the whole 10-step Euler loop of the 300M expert (single observation) as ONE
// cooperative launch of one CTA per SM, replacing ~930 per-operator launches.
//
// Decomposition (reference loop: pi0_infer.py:1165-1230, pi05_infer.py:418-523):
//   * every GEMM is partitioned over OUTPUT FEATURES with the full K per CTA (8-feature tiles, the n8 of
//     mma.sync.m16n8k16): no split-K exchange, no cluster.  The <= 56 suffix tokens are the M dimension (m16 tiles).
//   * each CTA's weights are pre-packed at load time into ONE contiguous stream of 16 KB chunks (8 features x 1024 K in
//     mma B-fragment order) in exactly the order the CTA consumes them; warp 8 copies the stream into a ring of shared
//     memory slots with cp.async.bulk, decoupled from the phase structure: while the CTA waits at a grid barrier the
//     weights of the next operators keep arriving from HBM.
//   * the GeGLU phase runs on tcgen05 instead: its chunks are K eighths of all eight (gate, up) tiles in the K-major,
//     128-byte-swizzled operand layout, the accumulator (128 x 64 fp32) lives in tensor memory, one lane issues the
//     MMAs on the TMA-written activation tiles and the epilogue reads one token row per thread (see phase_geglu).
//   * activations are small (<= 56 x 4096 bf16) and live in L2; warp 9 brings them in with TMA (cp.async.bulk.tensor,
//     128-byte swizzle, 64-wide K blocks) through a ring of four 256-wide K stages as soon as the grid barrier before
//     the phase is passed; the MMA warps read them with ldmatrix.
//   * phases are separated by grid barriers (one global counter, red.release / ld.acquire, ~1.1 us for 148 CTAs);
//     every spin is bounded by %globaltimer and raises the status word instead of hanging.
//   * the fp32 residual stream is owned by feature: CTA c < 128 keeps x[:, 8c..8c+7] in its shared memory for the whole
//     kernel; what other CTAs read is the bf16 mirror (GEMM operand) and per-CTA partial sums of squares (the RMS
//     norms are folded into the consuming GEMMs: norm(x) @ W = f * (x @ W), pi0_infer.py:1005; Pi05 adaRMS as
//     f * ((x * (1 + scale)) @ W) + shift @ W, pi05_infer.py:78-113).
//   * suffix attention (<= 448 query rows x <= 1024 keys, head dim 256): 32-row blocks x key splits over the CTAs,
//     single-pass softmax per split, partial outputs merged in a second short phase.
#pragma once
#include "common.cuh"

namespace xp {

constexpr int THREADS = 320;          // 8 MMA warps + weight-stream warp + activation (TMA) warp
constexpr int CTHREADS = 256;
constexpr int CHUNK_BYTES = 16384;    // 8 features x 1024 K, bf16, fragment order
constexpr int NSLOT = 6;
constexpr int MAX_ROWS = 56;          // suffix tokens held in shared memory
constexpr int TILE_BYTES = MAX_ROWS * 128;        // one 64-wide K block of the activation rows (TMA box, 128B swizzle)
constexpr int STAGE_BYTES = 4 * TILE_BYTES;       // 256 K
constexpr int N_ASTAGE = 4;
constexpr int A_BYTES = N_ASTAGE * STAGE_BYTES;   // 114688: activation stages / K, V and Q tiles of the attention
constexpr int SCR_BYTES = 8192;                   // GEMM: K-half exchange; attention: probabilities and row statistics
constexpr int RING_OFF = A_BYTES + SCR_BYTES;
constexpr int PERSIST_OFF = RING_OFF + NSLOT * CHUNK_BYTES;
constexpr int MAX_SEQ = 500;              // weight chunks per Euler step and CTA (the order list in shared memory)
constexpr int PERSIST_BYTES = 10240;          // barriers, per-token scales, this CTA's stream slice, rotary table of its QKV tiles
constexpr int SMEM_BYTES = PERSIST_OFF + PERSIST_BYTES + 1024;   // + slack to align the base to 1024 B
constexpr float SSQ_FIX = 16777216.0f;   // sums of squares travel as 40.24 fixed point: integer adds are order independent
constexpr int N_OWNERS = 128;         // CTAs that own 8 features of the 1024-wide stream / 32 hidden features
constexpr int CH_PER_LAYER = 17;      // stream slots per layer: qkv 0-2, o 3-4, gate/up K eighths 5-12, down 13-16
constexpr int ATT_ROWS = 32;          // query rows per attention work item
constexpr int ATT_MAX_KEYS = 96;      // keys per split
constexpr int MRG_BATCH = 12;         // key splits merged per round of loads
constexpr int ATT_V_OFF = ATT_MAX_KEYS * 512;     // V tiles behind the K tiles
constexpr int ATT_Q_OFF = 2 * ATT_MAX_KEYS * 512; // Q tiles (16 KB) fill the rest of the activation region

struct Params {
  // all maps are 3-D (64 elements, rows, 64-wide blocks of the row), 128-byte swizzle: one copy brings [block][row][128 B]
  CUtensorMap tm_xb;      // bf16 mirror of the stream [S, 1024], box 64 x MAX_ROWS x 4
  CUtensorMap tm_act;     // Pi0 action MLP input [C, 1024], same box
  CUtensorMap tm_attn;    // attention output [S, 2048], box 64 x S
  CUtensorMap tm_hidden;  // MLP hidden [S, 4096], box 64 x S
  CUtensorMap tm_q;       // queries as [S * 8, 256], box 64 x 32 x 4
  CUtensorMap tm_k;       // key cache [layers * T, 256], box 64 x att_kps x 4
  CUtensorMap tm_v;       // value cache, same
  int pi05, S, C, P, T, nl, nsteps, G;
  int att_nrb, att_ks, att_kps;   // row blocks, key splits, keys per split (multiple of 16, <= ATT_MAX_KEYS)
  const uint4* wstream;           // [G][chunks_per_cta][1024] uint4
  int chunks_per_cta;             // layers * CH_PER_LAYER + 2   (misc: +0 action MLP (Pi0), +1 out projection)
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
  bf16* noise; float* noise_f32; bf16* act; float* x_out; bf16* xb;
  unsigned long long* ssq;        // [3][64] per-token sums of squares of the stream, fixed point, rotating buffers (zeroed with bar_ctr)
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
// 16-byte global -> shared copy through L2 only
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
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
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
// Byte offset, inside a tile of 128-byte rows written by TMA with the 128-byte swizzle (tile base 1024-aligned), of the
// 16-byte chunk `ch` (0..7) of row `row`.
__host__ __device__ __forceinline__ uint32_t swz128(int row, int ch) { return (uint32_t)(row * 128 + ((ch ^ (row & 7)) << 4)); }

// ---- shared state ------------------------------------------------------------------------------------------------------
struct Ctx {
  const Params* p;
  uint32_t sbase;         // shared address of the activation region (1024-aligned)
  uint8_t* sptr;          // generic pointer to the same
  uint32_t w_full, w_empty, a_full, a_empty, att_full, att_full_v;   // att_full: Q and K tiles, att_full_v: V tiles
  uint32_t umma_bar;      // [8] completion of the GeGLU phase's tcgen05 MMAs, one per weight chunk
  uint32_t tmem;          // tensor-memory address of the GeGLU accumulator (64 columns)
  unsigned int umma_n;    // GeGLU phases run so far
  volatile int* go_count; // grid barriers passed, published by thread 0 for the activation warp
  volatile int* s_abort;
  float* fs;              // [64] per-token RMS scale
  float* xs;              // [64][8] this CTA's slice of the residual stream
  float* sttok;           // [8]
  float2* rope;           // [3 tiles][4 pairs][64 rows] (cos, sin) of this CTA's QKV features at the suffix positions
  unsigned int pk;        // residual-stream producer phases completed (selects the sum-of-squares buffer)
  unsigned int chunk_g;   // weight chunks consumed so far
  unsigned int a_g;       // activation stages consumed so far
  unsigned int att_n;     // attention phases run so far
  unsigned int bar_epoch; // grid barriers passed
  int cta, warp, lane, tid;
  int valid_len, pos_base;
  bool fine;
  int nmark;
};

// development timeline inside phases (CTA 0, Euler step 0, layer 1 only): append-only logs of (id << 48 | clock64),
// MMA thread 0 at trace[2560..], the activation warp at [3400..], the weight warp at [3700..]
#ifdef XP_FINE_TRACE
#define XP_LOG(c, base, cap, id) do { if ((c).fine && (c).nmark < (cap)) { (c).p->trace[(base) + (c).nmark] = ((unsigned long long)(id) << 48) | ((unsigned long long)clock64() & 0xffffffffffffull); ++(c).nmark; } } while (0)
#define XP_MARK(c, id) do { if ((c).tid == 0) XP_LOG(c, 2560, 800, id); } while (0)
#else
#define XP_LOG(c, base, cap, id) do {} while (0)
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
// bounded mbarrier wait; false = gave up (status word raised) or another CTA / role gave up.  (Kept inline: as separate
// functions the waiting loops cost 10 % of the kernel's time.)
__device__ __forceinline__ bool wait_bar_slow(uint32_t bar, uint32_t parity, volatile int* s_abort, unsigned int* bar_ctr, int* status) {
  const uint64_t t0 = globaltimer_ns();
  for (;;) {
    for (int i = 0; i < 128; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*s_abort) return false;
    if (*reinterpret_cast<volatile unsigned int*>(bar_ctr + 1)) { *s_abort = 1; return false; }
    if (globaltimer_ns() - t0 > VLA_WAIT_LIMIT_NS) {
      *s_abort = 1;
      atomicOr(bar_ctr + 1, 1u);
      atomicOr(status, VLA_ST_WAIT_TIMEOUT);
      return false;
    }
  }
}
__device__ __forceinline__ bool wait_bar(Ctx& c, uint32_t bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  return wait_bar_slow(bar, parity, c.s_abort, c.p->bar_ctr, c.p->status);
}
// bounded wait of MMA thread 0 for the count of completed grid barriers that the activation warp publishes
__device__ __forceinline__ void go_wait_slow(volatile int* go, int need, volatile int* s_abort, unsigned int* bar_ctr, int* status) {
  const uint64_t t0 = globaltimer_ns();
  unsigned int spins = 0;
  while (*go < need) {
    if ((++spins & 1023u) == 0) {
      if (*s_abort) return;
      if (*reinterpret_cast<volatile unsigned int*>(bar_ctr + 1)) { *s_abort = 1; return; }
      if (globaltimer_ns() - t0 > VLA_WAIT_LIMIT_NS) {
        *s_abort = 1;
        atomicOr(bar_ctr + 1, 1u);
        atomicOr(status, VLA_ST_WAIT_TIMEOUT);
        return;
      }
    }
  }
}
// shared address of the ring slot holding the g-th weight chunk, after waiting for it
__device__ __forceinline__ uint32_t acquire_chunk(Ctx& c, unsigned int g, bool* ok) {
  const unsigned int s = g % NSLOT;
  if (!wait_bar(c, c.w_full + 8 * s, (g / NSLOT) & 1u)) *ok = false;
  return c.sbase + RING_OFF + s * CHUNK_BYTES;
}
__device__ __forceinline__ void release_chunk(Ctx& c, unsigned int g) {
  __syncwarp();
  if (c.lane == 0) mbar_arrive(c.w_empty + 8 * (g % NSLOT));
}
// activation stage g of the ring (256 K of all rows): wait / hand back
__device__ __forceinline__ bool a_wait(Ctx& c, unsigned int g) { return wait_bar(c, c.a_full + 8 * (g & 3u), (g >> 2) & 1u); }
__device__ __forceinline__ void a_release(Ctx& c, unsigned int g) {
  __syncwarp();
  if (c.lane == 0) mbar_arrive(c.a_empty + 8 * (g & 3u));
}

// Grid-wide barrier of the MMA warps of all CTAs.  Thread 0 arrives on the global counter; the activation warp is the
// CTA's only poller of that counter (one poller per CTA keeps the L2 slice that holds it responsive): it publishes the
// number of completed barriers in shared memory and at once issues the next phase's loads.  Returns false after a
// timeout / abort (the same value in every MMA thread).
__device__ __forceinline__ bool grid_barrier(Ctx& c, int trace_slot) {
  cbar();
  ++c.bar_epoch;
  if (c.tid == 0) {
    const Params& p = *c.p;
    if (p.trace && c.cta == 0) p.trace[2 * trace_slot] = globaltimer_ns();
    // the release is cumulative over what the CTA barrier above ordered before it: no separate fence (one costs 0.3 us here)
    XP_LOG(c, 2560, 800, 98);
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.bar_ctr) : "memory");
    XP_LOG(c, 2560, 800, 99);
    if (*c.go_count < (int)c.bar_epoch) go_wait_slow(c.go_count, (int)c.bar_epoch, c.s_abort, p.bar_ctr, p.status);
    __threadfence_block();   // the loader's acquire at GPU scope, its store of the count, this read and the barrier below form the chain
    if (p.trace && c.cta == 0) p.trace[2 * trace_slot + 1] = globaltimer_ns();
  }
  cbar();
  return *c.s_abort == 0;
}

// Per-token RMS scale: the owners of the stream add their partial sums of squares (fixed point) into one word per token
// with integer atomics, so the sum does not depend on the order; fs[t] = rsqrt(ssq[t] / 1024 + 1e-6).
// The load is issued at the start of a phase and consumed after its MMAs.
__device__ __forceinline__ unsigned long long fs_issue(const Ctx& c) {
  return c.tid < 64 ? __ldcg(c.p->ssq + ((c.pk + 2u) % 3u) * 64 + c.tid) : 0ull;   // buffer of producer phase pk - 1
}
__device__ __forceinline__ void fs_finish(Ctx& c, unsigned long long v) {
  if (c.tid < 64) c.fs[c.tid] = rsqrtf((float)v * (1.0f / (SSQ_FIX * 1024.0f)) + 1e-6f);
}
// producer side: called once per producer phase by every MMA thread of every CTA
__device__ __forceinline__ void ssq_rotate(Ctx& c) {
  if (c.cta == 0 && c.tid < 64) c.p->ssq[((c.pk + 1u) % 3u) * 64 + c.tid] = 0ull;   // next phase's buffer, idle since two phases
}
__device__ __forceinline__ void ssq_add(const Ctx& c, int token, float sq) {
  atomicAdd(c.p->ssq + (c.pk % 3u) * 64 + token, (unsigned long long)__float2ull_rn(sq * SSQ_FIX));
}

// ---- GEMM cores ------------------------------------------------------------------------------------------------------------
// NT feature tiles (their chunks at slot addresses sl[0..NT-1]) against the four activation stages a_g0..a_g0+3 (K = 1024);
// warp (mi, kh) takes rows 16 mi.. and K half kh.  The loop is bound by shared-memory bandwidth (1 KB of A and NT x 512 B
// of B per iteration and warp), so the more tiles share an A fragment the better.
template <int NT>
__device__ __forceinline__ void mma_resident(Ctx& c, const uint32_t* sl, int rows, unsigned int a_g0, float (&acc)[NT][4], bool* ok,
                                             int nt = NT) {
  const int mi = c.warp & 3, kh = c.warp >> 2;
  float acc2[4] = {0.f, 0.f, 0.f, 0.f};   // a single tile alternates two accumulators to break the dependent chain
#pragma unroll
  for (int t = 0; t < NT; ++t)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[t][j] = 0.f;
  // every warp waits for the stages of its K half, also a warp without rows: the stages are then handed back in step
  if (!a_wait(c, a_g0 + 2 * kh) || !a_wait(c, a_g0 + 2 * kh + 1)) *ok = false;
  XP_MARK(c, 90);
  if (16 * mi >= rows || !*ok) return;
  const int row = min(16 * mi + (c.lane & 15), rows - 1);
  const int hi = c.lane >> 4;
  const uint32_t lane_off = (uint32_t)c.lane * 16;
  const uint32_t a_off0 = swz128(row, hi), a_off1 = swz128(row, hi + 2), a_off2 = swz128(row, hi + 4), a_off3 = swz128(row, hi + 6);
#pragma unroll 2
  for (int i = 0; i < 8; ++i) {          // one 64-wide K block (four k16 steps) per round
    const int kb = 8 * kh + i;
    const uint32_t tile = c.sbase + (uint32_t)((a_g0 + (kb >> 2)) & 3u) * STAGE_BYTES + (uint32_t)(kb & 3) * TILE_BYTES;
    uint32_t a[16];
    ldsm_x4(tile + a_off0, a[0], a[1], a[2], a[3]);
    ldsm_x4(tile + a_off1, a[4], a[5], a[6], a[7]);
    ldsm_x4(tile + a_off2, a[8], a[9], a[10], a[11]);
    ldsm_x4(tile + a_off3, a[12], a[13], a[14], a[15]);
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      if (t >= nt) break;                // fewer tiles than NT: the same in every thread
      const uint32_t baddr = sl[t] + (uint32_t)(2 * kb) * 512 + lane_off;
      const uint4 b0 = lds128(baddr);
      const uint4 b1 = lds128(baddr + 512);
      float* second = NT == 1 ? acc2 : acc[t];
      mma16816(acc[t], a[0], a[1], a[2], a[3], b0.x, b0.y);
      mma16816(second, a[4], a[5], a[6], a[7], b0.z, b0.w);
      mma16816(acc[t], a[8], a[9], a[10], a[11], b1.x, b1.y);
      mma16816(second, a[12], a[13], a[14], a[15], b1.z, b1.w);
    }
  }
  if (NT == 1) {
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[0][j] += acc2[j];
  }
}
// every warp hands the four stages of a K = 1024 phase back
__device__ __forceinline__ void a_release4(Ctx& c) {
  __syncwarp();
  if (c.lane == 0)
    for (int s = 0; s < 4; ++s) mbar_arrive(c.a_empty + 8 * ((c.a_g + s) & 3u));
  c.a_g += 4;
}

// Adds the partial accumulators of the K-half-1 warps to those of the K-half-0 warps through shared memory (8 KB:
// [mi (4)][tile (4)][lane (32)] float4).  After the call the warps with kh == 0 hold the sums.  A second call within
// one phase passes pre_sync: the extra barrier keeps its writes behind the reads of the first call.
template <int NT>
__device__ __forceinline__ void reduce_khalves(const Ctx& c, bool pre_sync, float (&acc)[NT][4]) {
  static_assert(NT <= 4, "the exchange area holds four tiles per warp");
  const int mi = c.warp & 3, kh = c.warp >> 2;
  float4* red = reinterpret_cast<float4*>(c.sptr + A_BYTES) + mi * 128 + c.lane;
  if (pre_sync) cbar();
  if (kh == 1) {
#pragma unroll
    for (int t = 0; t < NT; ++t) red[t * 32] = make_float4(acc[t][0], acc[t][1], acc[t][2], acc[t][3]);
  }
  cbar();
  if (kh == 0) {
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      const float4 v = red[t * 32];
      acc[t][0] += v.x; acc[t][1] += v.y; acc[t][2] += v.z; acc[t][3] += v.w;
    }
  }
}

// One feature tile (weight chunks chunk_g .. chunk_g + K/1024 - 1) against K/256 activation stages streamed through the ring.
__device__ __forceinline__ bool mma_streamed(Ctx& c, int rows, int K, float (&acc)[1][4]) {
  const int mi = c.warp & 3, kh = c.warp >> 2;
  const int n_stages = K >> 8;
  bool ok = true;
  float acc2[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int j = 0; j < 4; ++j) acc[0][j] = 0.f;
  const bool active = 16 * mi < rows;
  const int row = min(16 * mi + (c.lane & 15), rows - 1);
  const int hi = c.lane >> 4;
  uint32_t slot = 0;
  for (int st = 0; st < n_stages; ++st) {
    const unsigned int g = c.a_g + st;
    if ((st & 3) == 0) slot = acquire_chunk(c, c.chunk_g + (st >> 2), &ok);
    if (!a_wait(c, g)) ok = false;   // also a warp without rows: keeps the hand-back of the stages in step
    if (active) {
      if (ok) {
        const uint32_t stage = c.sbase + (uint32_t)(g & 3u) * STAGE_BYTES;
        const uint32_t bsrc = slot + (uint32_t)(((st & 3) * 8 + 4 * kh) * 32 + c.lane) * 16;
        uint4 b[4];
        uint32_t a[4][8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {      // all fragment loads of the stage first, then its eight MMAs
          const int spl = 4 * kh + i;
          b[i] = lds128(bsrc + i * 512);
          const uint32_t tile = stage + (uint32_t)(spl >> 1) * TILE_BYTES;
          const int c0 = 4 * (spl & 1) + hi;
          ldsm_x4(tile + swz128(row, c0), a[i][0], a[i][1], a[i][2], a[i][3]);
          ldsm_x4(tile + swz128(row, c0 + 2), a[i][4], a[i][5], a[i][6], a[i][7]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          mma16816(acc[0], a[i][0], a[i][1], a[i][2], a[i][3], b[i].x, b[i].y);
          mma16816(acc2, a[i][4], a[i][5], a[i][6], a[i][7], b[i].z, b[i].w);
        }
      }
    }
    a_release(c, g);
    XP_MARK(c, 91);
    if ((st & 3) == 3) release_chunk(c, c.chunk_g + (st >> 2));
  }
  c.a_g += (unsigned int)n_stages;
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
  bool store_x;      // also write the fp32 stream to global memory (nothing in the kernel reads it: only the state after the
                     // last layer of a step is kept for inspection)
  float b0, b1, g0, g1, m0, m1;   // bias, gate and mirror scale (1 + adaRMS scale of the consuming norm) of features n, n+1
};
__device__ __forceinline__ ResidEpi make_resid(Ctx& c, int rows, int row_off, bool accumulate, const float* bias, const float* gate,
                                               const float* mscale) {
  const int n = 8 * c.cta + 2 * (c.lane & 3);
  ResidEpi e;
  e.rows = rows; e.row_off = row_off; e.accumulate = accumulate; e.store_x = false;
  e.b0 = bias ? bias[n] : 0.f; e.b1 = bias ? bias[n + 1] : 0.f;
  e.g0 = gate ? gate[n] : 1.f; e.g1 = gate ? gate[n + 1] : 1.f;
  e.m0 = mscale ? 1.f + mscale[n] : 1.f; e.m1 = mscale ? 1.f + mscale[n + 1] : 1.f;
  return e;
}
// residual-stream update for this CTA's 8 features; writes the bf16 mirror, the fp32 copy and the partial sums of squares
__device__ __forceinline__ void epi_resid(Ctx& c, const ResidEpi& e, const float* acc) {
  const Params& p = *c.p;
  const int mi = c.warp & 3;
  const int j0 = 2 * (c.lane & 3), n = 8 * c.cta + j0;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = 16 * mi + (c.lane >> 2) + 8 * h;
    const bool valid = r < e.rows;
    const int t = r + e.row_off;
    float v0 = 0.f, v1 = 0.f;
    if (valid) {
      if (e.accumulate) {
        v0 = c.xs[t * 8 + j0] + e.g0 * acc[2 * h];
        v1 = c.xs[t * 8 + j0 + 1] + e.g1 * acc[2 * h + 1];
      } else {
        v0 = acc[2 * h] + e.b0;
        v1 = acc[2 * h + 1] + e.b1;
      }
      c.xs[t * 8 + j0] = v0;
      c.xs[t * 8 + j0 + 1] = v1;
      *reinterpret_cast<uint32_t*>(p.xb + (size_t)t * 1024 + n) = pack_bf16x2(v0 * e.m0, v1 * e.m1);
      if (e.store_x) *reinterpret_cast<float2*>(p.x_out + (size_t)t * 1024 + n) = make_float2(v0, v1);
    }
    float sq = v0 * v0 + v1 * v1;
    sq += __shfl_xor_sync(0xffffffffu, sq, 1);
    sq += __shfl_xor_sync(0xffffffffu, sq, 2);
    if (valid && (c.lane & 3) == 0) ssq_add(c, t, sq);
  }
}

// ---- phases ----------------------------------------------------------------------------------------------------------------
// Action in-projection (K = 32) straight from global weights: Pi0 -> act = silu(noise @ W + time_bias[step]);
// Pi05 -> x = noise @ W + b (start of the residual stream).  CTA c < 128 owns features 8c..8c+7.  The 50 x 32 noise
// tile is brought in by the MMA threads themselves (the activation ring is idle between phases).
__device__ __forceinline__ void phase_in_proj(Ctx& c, int step) {
  const Params& p = *c.p;
  if (p.pi05) ssq_rotate(c);
  if (c.cta >= N_OWNERS) { if (p.pi05) ++c.pk; return; }
  for (int idx = c.tid; idx < p.C * 4; idx += CTHREADS) {
    const int row = idx >> 2, ch = idx & 3;
    cp_async16(c.sbase + swz128(row, ch), p.noise + (size_t)row * 32 + ch * 8);
  }
  cp_async_commit();
  const int mi = c.warp & 3, kh = c.warp >> 2;
  const int j0 = 2 * (c.lane & 3), n = 8 * c.cta + j0;
  float b0 = 0.f, b1 = 0.f;
  ResidEpi e;
  if (!p.pi05) {
    const float* tb = p.b_in + (size_t)step * p.ld_b_in;
    b0 = tb[n]; b1 = tb[n + 1];
  } else {
    e = make_resid(c, p.C, 0, false, p.b_in, nullptr, p.style_attn + (size_t)step * p.nl * 3072);   // pre-attention norm of layer 0
  }
  const int nb = 8 * c.cta + (c.lane >> 2);
  uint32_t wb[2][2];
#pragma unroll
  for (int s = 0; s < 2; ++s) {
    const bf16* w = p.w_in + (size_t)nb * 64 + 16 * s + 2 * (c.lane & 3);
    wb[s][0] = *reinterpret_cast<const uint32_t*>(w);
    wb[s][1] = *reinterpret_cast<const uint32_t*>(w + 8);
  }
  cp_async_wait<0>();
  cbar();
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  if (kh == 0 && 16 * mi < p.C) {
    const int row = min(16 * mi + (c.lane & 15), p.C - 1);
    const int hi = c.lane >> 4;
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      uint32_t a0, a1, a2, a3;
      ldsm_x4(c.sbase + swz128(row, 2 * s + hi), a0, a1, a2, a3);
      mma16816(acc, a0, a1, a2, a3, wb[s][0], wb[s][1]);
    }
  }
  if (kh == 0) {
    if (!p.pi05) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int r = 16 * mi + (c.lane >> 2) + 8 * h;
        if (r < p.C)
          *reinterpret_cast<uint32_t*>(p.act + (size_t)r * 1024 + n) = pack_bf16x2(silu_f(acc[2 * h] + b0), silu_f(acc[2 * h + 1] + b1));
      }
    } else {
      epi_resid(c, e, acc);
    }
  }
  if (p.pi05) ++c.pk;
}

// Pi0 action MLP: x[1 + a] = act[a] @ W + b; x[0] = state token.
__device__ __forceinline__ bool phase_action_mlp(Ctx& c) {
  const Params& p = *c.p;
  ssq_rotate(c);
  if (c.cta >= N_OWNERS) { ++c.pk; return true; }
  bool ok = true;
  const ResidEpi e = make_resid(c, p.C, 1, false, p.b_mlp, nullptr, nullptr);
  const uint32_t sl = acquire_chunk(c, c.chunk_g, &ok);
  float acc[1][4];
  mma_resident<1>(c, &sl, p.C, c.a_g, acc, &ok);
  release_chunk(c, c.chunk_g);
  a_release4(c);
  c.chunk_g += 1;
  reduce_khalves<1>(c, false, acc);
  if ((c.warp >> 2) == 0) epi_resid(c, e, acc[0]);
  if (c.tid < 8) {   // the state token row (constant over the Euler steps)
    const float v = c.sttok[c.tid];
    c.xs[c.tid] = v;
    p.xb[8 * c.cta + c.tid] = __float2bfloat16(v);
    float sq = v * v;
    sq += __shfl_xor_sync(0xffu, sq, 1);
    sq += __shfl_xor_sync(0xffu, sq, 2);
    sq += __shfl_xor_sync(0xffu, sq, 4);
    if (c.tid == 0) ssq_add(c, 0, sq);
  }
  ++c.pk;
  return ok;
}

// QKV projection with folded norm, rotary embedding and K/V-cache append (pi0_infer.py:777-810).
// CTA c owns feature tiles c, c + G, c + 2G (< 320).
__device__ __forceinline__ int qkv_tile_count(int cta, int G) {
  return (cta + 2 * G < 320) ? 3 : ((cta + G < 320) ? 2 : (cta < 320 ? 1 : 0));
}
__device__ __forceinline__ bool phase_qkv(Ctx& c, int step, int layer) {
  constexpr int NQ = 3;
  const Params& p = *c.p;
  const int nq = qkv_tile_count(c.cta, p.G);   // tiles of this CTA (<= NQ); one instantiation serves every count
  if (nq == 0) return true;
  XP_MARK(c, 0);
  bool ok = true;
  const int mi = c.warp & 3, kh = c.warp >> 2;
  // the few values the epilogue needs from global memory are requested before the MMAs
  float bias[NQ][2];
#pragma unroll
  for (int t = 0; t < NQ; ++t) { bias[t][0] = 0.f; bias[t][1] = 0.f; }
  if (p.pi05 && kh == 0) {
    const float* bsrc = p.sw_qkv + ((size_t)step * p.nl + layer) * 2560;
#pragma unroll
    for (int t = 0; t < NQ; ++t) {
      if (t >= nq) break;
      const int n = 8 * (c.cta + t * p.G) + 2 * (c.lane & 3);
      bias[t][0] = bsrc[n];
      bias[t][1] = bsrc[n + 1];
    }
  }
  const unsigned long long fv = fs_issue(c);
  uint32_t sl[NQ];
#pragma unroll
  for (int j = 0; j < NQ; ++j) sl[j] = j < nq ? acquire_chunk(c, c.chunk_g + j, &ok) : 0u;
  XP_MARK(c, 1);
  float acc[NQ][4];
  mma_resident<NQ>(c, sl, p.S, c.a_g, acc, &ok, nq);
  XP_MARK(c, 2);
#pragma unroll
  for (int j = 0; j < NQ; ++j)
    if (j < nq) release_chunk(c, c.chunk_g + j);
  a_release4(c);
  c.chunk_g += nq;
  fs_finish(c, fv);
  reduce_khalves<NQ>(c, false, acc);   // the barrier inside also publishes fs
  XP_MARK(c, 3);
  if (kh == 0) {
    bf16* kc = p.kcache + (size_t)layer * p.T * 256;
    bf16* vc = p.vcache + (size_t)layer * p.T * 256;
#pragma unroll
    for (int t = 0; t < NQ; ++t) {
      if (t >= nq) break;
      const int n = 8 * (c.cta + t * p.G) + 2 * (c.lane & 3);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int r = 16 * mi + (c.lane >> 2) + 8 * h;
        if (r >= p.S) continue;
        const float f = c.fs[r];
        const float v0 = f * acc[t][2 * h] + bias[t][0], v1 = f * acc[t][2 * h + 1] + bias[t][1];
        const float2 cssn = c.rope[(t * 4 + (c.lane & 3)) * 64 + r];
        const uint32_t o = pack_bf16x2(v0 * cssn.x - v1 * cssn.y, v1 * cssn.x + v0 * cssn.y);
        if (n < 2048) *reinterpret_cast<uint32_t*>(p.q + (size_t)r * 2048 + n) = o;
        else if (n < 2304) *reinterpret_cast<uint32_t*>(kc + (size_t)(p.P + r) * 256 + (n - 2048)) = o;
        else *reinterpret_cast<uint32_t*>(vc + (size_t)(p.P + r) * 256 + (n - 2304)) = o;
      }
    }
  }
  XP_MARK(c, 4);
  return ok;
}

// GeGLU: hidden[:, 32c..32c+31] = gelu(f * (xb @ Wg) + bg) * (f * (xb @ Wu) + bu), four (gate, up) tile pairs per CTA.
// This phase runs on tcgen05: with mma.sync every activation fragment is re-read from shared memory for each group of
// four feature tiles and the loop sat on the shared-memory bandwidth limit; the tensor core reads both operands
// straight from the TMA-written tiles, each once.  The CTA's eight weight chunks of the layer are K eighths of all
// eight tiles ([K block (2)][row (64) = per pair: gate 8 | up 8][128 B, 128-byte swizzle]), so that one accumulator of
// 64 columns takes the whole phase: lane 0 of warp 2 (a warp without epilogue rows) issues, per 64-wide K block, four
// MMAs of M = 128 (the 56 token rows of the activation tile; rows 56..127 read whatever lies behind the tile and their
// results are never looked at) x N = 64 x K = 16 as chunks and activation stages arrive, and commits per chunk; the other
// warps hand each chunk back when its commit has landed (warp 3 also on the issuer's behalf), and warps 0, 1, 4, 5
// (TMEM lane quarters 0 and 1 = token rows 0..63, two column halves) run the epilogue with one token row per thread.
__device__ __forceinline__ bool phase_geglu(Ctx& c, int step, int layer) {
  const Params& p = *c.p;
  if (c.cta >= N_OWNERS) return true;
  bool ok = true;
  XP_MARK(c, 60);
  const int qtr = c.warp & 3, half = c.warp >> 2;
  const int r = 32 * qtr + c.lane;                       // token row of this thread in the epilogue
  const bool epi = qtr < 2;
  const uint32_t par = c.umma_n & 1u;
  ++c.umma_n;
  if (c.warp == 2) {
    if (c.lane == 0) {
      // instruction descriptor: D = f32, A = B = bf16, both K-major, N = 64, M = 128
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((64u >> 3) << 17) | (8u << 24);
      int j = 0;
      for (; j < 8; ++j) {
        const uint32_t slot = acquire_chunk(c, c.chunk_g + j, &ok);
        if ((j & 1) == 0 && !a_wait(c, c.a_g + (j >> 1))) ok = false;
        if (!ok) break;
        tc_fence_after();
        const uint32_t stage = c.sbase + (uint32_t)((c.a_g + (j >> 1)) & 3u) * STAGE_BYTES;
#pragma unroll
        for (int kb = 0; kb < 2; ++kb) {
          const uint64_t da = attn_desc_sw128(stage + (2 * (j & 1) + kb) * TILE_BYTES), db = attn_desc_sw128(slot + kb * 8192);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) umma_bf16(c.tmem, da + 2 * kk, db + 2 * kk, idesc, (j | kb | kk) != 0 ? 1u : 0u);
        }
        umma_commit(c.umma_bar + 8 * j);   // this chunk has been read once its MMAs complete: the ring refills during the phase
      }
      // after a failed wait the remaining commits are still made: the other warps are released and see the abort flag
      for (int k = j; k < 8; ++k) umma_commit(c.umma_bar + 8 * k);
      // the issuing lane never waits for a commit (that would tie the issue of a chunk to the completion of the one
      // before it); warp 3 hands the chunks back on this warp's behalf
    }
    __syncwarp();
  } else {
    // the per-token scale of this thread's row, straight from the sums of squares (no exchange through shared memory)
    unsigned long long ssq = 0ull;
    if (epi && r < p.S) ssq = __ldcg(p.ssq + ((c.pk + 2u) % 3u) * 64 + r);
    float bg[2][8], bu[2][8];
#pragma unroll
    for (int q = 0; q < 2; ++q)
#pragma unroll
      for (int k = 0; k < 8; ++k) { bg[q][k] = 0.f; bu[q][k] = 0.f; }
    const int n0 = 32 * c.cta + 16 * half;               // first of this thread's sixteen hidden features (two tile pairs)
    if (p.pi05 && epi) {
      const float* g = p.sw_gate + ((size_t)step * p.nl + layer) * 4096 + n0;
      const float* u = p.sw_up + ((size_t)step * p.nl + layer) * 4096 + n0;
#pragma unroll
      for (int q = 0; q < 2; ++q)
#pragma unroll
        for (int k = 0; k < 8; ++k) { bg[q][k] = g[8 * q + k]; bu[q][k] = u[8 * q + k]; }
    }
    for (int j = 0; j < 8; ++j) {
      if (!wait_bar(c, c.umma_bar + 8 * j, par)) ok = false;
      release_chunk(c, c.chunk_g + j);
      if (c.warp == 3 && c.lane == 0) mbar_arrive(c.w_empty + 8 * ((c.chunk_g + j) % NSLOT));   // for the issuing warp
    }
    tc_fence_after();
    XP_MARK(c, 61);
    if (epi) {
      uint32_t v[32];
      tmem_ld32(c.tmem + ((uint32_t)(32 * qtr) << 16) + 32 * half, v);   // pairs 2 half, 2 half + 1: gate 8 | up 8 each
      tmem_ld_wait();
      if (r < p.S && ok) {
        const float f = rsqrtf((float)ssq * (1.0f / (SSQ_FIX * 1024.0f)) + 1e-6f);
        uint32_t o[8];
#pragma unroll
        for (int q = 0; q < 2; ++q)
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float h0 = gelu_tanh_f(f * __uint_as_float(v[16 * q + 2 * k]) + bg[q][2 * k]) * (f * __uint_as_float(v[16 * q + 8 + 2 * k]) + bu[q][2 * k]);
            const float h1 = gelu_tanh_f(f * __uint_as_float(v[16 * q + 2 * k + 1]) + bg[q][2 * k + 1]) * (f * __uint_as_float(v[16 * q + 9 + 2 * k]) + bu[q][2 * k + 1]);
            o[4 * q + k] = pack_bf16x2(h0, h1);
          }
        uint4* dst = reinterpret_cast<uint4*>(p.hidden + (size_t)r * 4096 + n0);
        dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
        dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
      }
    }
  }
  c.chunk_g += 8;
  tc_fence_before();
  a_release4(c);
  XP_MARK(c, 65);
  return ok;
}

// Attention-out (K = 2048) and MLP-down (K = 4096) projections with the residual add.
__device__ __forceinline__ bool phase_resid(Ctx& c, int K, const float* gate, const float* mscale, bool store_x) {
  const Params& p = *c.p;
  ssq_rotate(c);
  if (c.cta >= N_OWNERS) { ++c.pk; return true; }
  XP_MARK(c, K == 2048 ? 20 : 40);
  ResidEpi e = make_resid(c, p.S, 0, true, nullptr, gate, mscale);
  e.store_x = store_x;
  float acc[1][4];
  const bool ok = mma_streamed(c, p.S, K, acc);
  XP_MARK(c, K == 2048 ? 21 : 41);
  reduce_khalves<1>(c, false, acc);
  if ((c.warp >> 2) == 0) epi_resid(c, e, acc[0]);
  XP_MARK(c, K == 2048 ? 22 : 42);
  ++c.pk;
  return ok;
}

// Out projection + Euler update: noise += f * (xb[action rows] @ W_out) + b  (pi0_infer.py:1224-1230).  CTA c < 4.
__device__ __forceinline__ bool phase_out(Ctx& c, int step) {
  const Params& p = *c.p;
  if (c.cta >= 4) return true;
  bool ok = true;
  const int off = p.pi05 ? 0 : 1;
  const unsigned long long fv = fs_issue(c);
  const uint32_t sl = acquire_chunk(c, c.chunk_g, &ok);
  float acc[1][4];
  mma_resident<1>(c, &sl, p.C, c.a_g, acc, &ok);
  release_chunk(c, c.chunk_g);
  a_release4(c);
  c.chunk_g += 1;
  fs_finish(c, fv);
  reduce_khalves<1>(c, false, acc);
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
// Shared memory: K tiles [4 dim blocks][kps keys][128 B] at 0, V tiles the same at ATT_V_OFF, Q tiles [4][32][128 B]
// at ATT_Q_OFF, all written by TMA with the 128-byte swizzle.
__device__ __forceinline__ bool phase_attention(Ctx& c, int layer) {
  const Params& p = *c.p;
  const int n_items = p.att_nrb * p.att_ks;
  if (c.cta >= n_items) return true;
  const int rb = c.cta / p.att_ks, sp = c.cta - rb * p.att_ks;
  const int R = p.S * 8;
  const int r0 = rb * ATT_ROWS;
  const int key0 = sp * p.att_kps;
  const int nk = max(0, min(p.att_kps, p.T - key0));          // real keys of this split
  const int nkp = (nk + 15) & ~15;                            // padded to the mma K step
  const uint32_t sQ = c.sbase + ATT_Q_OFF, sK = c.sbase, sV = c.sbase + ATT_V_OFF;
  const uint32_t kv_tile = (uint32_t)p.att_kps * 128;
  const uint32_t sP = c.sbase + A_BYTES;                      // bf16 [32][104] (pitch 208 B)
  float* red = reinterpret_cast<float*>(c.sptr + A_BYTES + 32 * 208);   // rmax[4][32], rsum[4][32]
  XP_MARK(c, 10);
  bool ok = wait_bar(c, c.att_full, c.att_n & 1u);   // Q and K; the V tiles are waited for in front of the PV product
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
  if (ok) {
    const int qrow = 16 * mi + (c.lane & 15);
    const int hi = c.lane >> 4;
    struct SF { uint32_t a[8]; uint32_t b[3][4]; };
    auto load = [&](SF& f, int k2) {     // two k16 steps (32 dims): dims block k2 >> 1, chunks 4 (k2 & 1) ..
      const uint32_t qt = sQ + (uint32_t)(k2 >> 1) * 4096;
      const int c0 = 4 * (k2 & 1) + hi;
      ldsm_x4(qt + swz128(qrow, c0), f.a[0], f.a[1], f.a[2], f.a[3]);
      ldsm_x4(qt + swz128(qrow, c0 + 2), f.a[4], f.a[5], f.a[6], f.a[7]);
#pragma unroll
      for (int t = 0; t < 3; ++t) {
        const int kt = grp + 4 * t;
        if (kt < n_kt) {
          const int krow = 8 * kt + (c.lane & 7);
          ldsm_x4(sK + (uint32_t)(k2 >> 1) * kv_tile + swz128(krow, 4 * (k2 & 1) + (c.lane >> 3)), f.b[t][0], f.b[t][1], f.b[t][2], f.b[t][3]);
        }
      }
    };
    auto mma = [&](const SF& f) {
#pragma unroll
      for (int t = 0; t < 3; ++t) {
        if (grp + 4 * t < n_kt) {
          mma16816(s[t], f.a[0], f.a[1], f.a[2], f.a[3], f.b[t][0], f.b[t][1]);
          mma16816(s[t], f.a[4], f.a[5], f.a[6], f.a[7], f.b[t][2], f.b[t][3]);
        }
      }
    };
    SF f0, f1;
    load(f0, 0);
#pragma unroll 1
    for (int k2 = 0; k2 < 8; k2 += 2) {
      load(f1, k2 + 1);
      mma(f0);
      if (k2 + 2 < 8) load(f0, k2 + 2);
      mma(f1);
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
  if (!wait_bar(c, c.att_full_v, c.att_n & 1u)) ok = false;
  ++c.att_n;
  // ---- O = P V for dims 64 grp .. 64 grp + 63 (one 64-dim V block per warp group) ----
  float o[8][4];
#pragma unroll
  for (int t = 0; t < 8; ++t)
#pragma unroll
    for (int j = 0; j < 4; ++j) o[t][j] = 0.f;
  if (ok) {
    const int prow = 16 * mi + (c.lane & 15);
    const uint32_t vt = sV + (uint32_t)grp * kv_tile;
    struct PF { uint32_t a[4]; uint32_t b[4][4]; };
    auto load = [&](PF& f, int ks) {
      ldsm_x4(sP + prow * 208 + (uint32_t)((2 * ks + (c.lane >> 4)) << 4), f.a[0], f.a[1], f.a[2], f.a[3]);
      const int vrow = 16 * ks + (c.lane & 7) + 8 * ((c.lane >> 3) & 1);
#pragma unroll
      for (int t2 = 0; t2 < 4; ++t2)     // two 8-dim tiles per ldmatrix
        ldsm_x4_t(vt + swz128(vrow, 2 * t2 + (c.lane >> 4)), f.b[t2][0], f.b[t2][1], f.b[t2][2], f.b[t2][3]);
    };
    auto mma = [&](const PF& f) {
#pragma unroll
      for (int t2 = 0; t2 < 4; ++t2) {
        mma16816(o[2 * t2], f.a[0], f.a[1], f.a[2], f.a[3], f.b[t2][0], f.b[t2][1]);
        mma16816(o[2 * t2 + 1], f.a[0], f.a[1], f.a[2], f.a[3], f.b[t2][2], f.b[t2][3]);
      }
    };
    const int n_ks = nkp >> 4;
    PF f0, f1;
    if (n_ks > 0) load(f0, 0);
#pragma unroll 1
    for (int ks = 0; ks < n_ks; ks += 2) {
      if (ks + 1 < n_ks) load(f1, ks + 1);
      mma(f0);
      if (ks + 2 < n_ks) load(f0, ks + 2);
      if (ks + 1 < n_ks) mma(f1);
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
  return ok;
}

// Suffix attention, part 2: rows are dealt round-robin to the CTAs; a warp pair merges one row (each lane 4 dims) over
// the key splits, with every load of a batch of MRG_BATCH splits issued before the first use (one L2 round trip for the
// usual 11 splits of 788 prefix + 51 suffix keys).
__device__ __forceinline__ void phase_attention_merge(Ctx& c) {
  const Params& p = *c.p;
  const int R = p.S * 8, ks = p.att_ks;
  const int slot = c.warp >> 1, half = c.warp & 1;
  XP_MARK(c, 16);
  for (int r = c.cta + slot * p.G; r < R; r += 4 * p.G) {
    const int rb = r / ATT_ROWS, rl = r - rb * ATT_ROWS;
    const float2* st = reinterpret_cast<const float2*>(p.att_stat) + (size_t)rb * ks * ATT_ROWS + rl;
    const float4* pt = reinterpret_cast<const float4*>(p.att_part + ((size_t)rb * ks * ATT_ROWS + rl) * 256 + 128 * half) + c.lane;
    float mx = -INFINITY, L = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = 0; s0 < ks; s0 += MRG_BATCH) {
      float2 sv[MRG_BATCH];
      float4 pv[MRG_BATCH];
#pragma unroll
      for (int i = 0; i < MRG_BATCH; ++i) {
        const bool in = s0 + i < ks;
        sv[i] = in ? __ldcg(st + (size_t)(s0 + i) * ATT_ROWS) : make_float2(-INFINITY, 0.f);
        pv[i] = in ? __ldcg(pt + (size_t)(s0 + i) * ATT_ROWS * 64) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
      float bm = mx;
#pragma unroll
      for (int i = 0; i < MRG_BATCH; ++i) bm = fmaxf(bm, sv[i].x);
      // rescale what has been accumulated so far to the new maximum (first batch: nothing accumulated, factor irrelevant)
      const float resc = (mx == -INFINITY) ? 0.f : exp2f(mx - bm);
      L *= resc; acc.x *= resc; acc.y *= resc; acc.z *= resc; acc.w *= resc;
      mx = bm;
#pragma unroll
      for (int i = 0; i < MRG_BATCH; ++i) {
        const float w = sv[i].x == -INFINITY ? 0.f : exp2f(sv[i].x - mx);
        L += w * sv[i].y;
        acc.x += w * pv[i].x; acc.y += w * pv[i].y; acc.z += w * pv[i].z; acc.w += w * pv[i].w;
      }
    }
    const float inv = 1.0f / L;
    uint2 o;
    o.x = pack_bf16x2(acc.x * inv, acc.y * inv);
    o.y = pack_bf16x2(acc.z * inv, acc.w * inv);
    *reinterpret_cast<uint2*>(p.attn + (size_t)r * 256 + 128 * half + 4 * c.lane) = o;
  }
  XP_MARK(c, 17);
}

// ---- weight stream (warp 8, one lane) ---------------------------------------------------------------------------------------
// The CTA's chunks in the order its phases consume them (the same order in every Euler step), copied into the ring as
// its slots are handed back.  (Requesting chunks into L2 ahead of the copy, cp.async.bulk.prefetch.L2, made the kernel
// 2.5 % slower and is not done.)
__device__ __forceinline__ void weight_producer_loop(Ctx& c) {
  const Params& p = *c.p;
  const uint4* base = p.wstream + (size_t)c.cta * p.chunks_per_cta * (CHUNK_BYTES / 16);
  const uint64_t pol = policy_evict_first();    // a chunk is read once per Euler step
  unsigned short* seq = reinterpret_cast<unsigned short*>(c.sptr + PERSIST_OFF + 9216);
  int n = 0;
  {
    auto range = [&](int first, int count) {
      for (int j = 0; j < count && n < MAX_SEQ; ++j) seq[n++] = (unsigned short)(first + j);
    };
    const int nq = qkv_tile_count(c.cta, p.G);
    const bool owner = c.cta < N_OWNERS;
    if (!p.pi05 && owner) range(p.misc_base, 1);
    for (int l = 0; l < p.nl; ++l) {
      range(l * CH_PER_LAYER, nq);
      if (owner) range(l * CH_PER_LAYER + 3, CH_PER_LAYER - 3);   // attention-out, GeGLU quarters, down
    }
    if (c.cta < 4) range(p.misc_base + 1, 1);
  }
  const long long total = (long long)n * p.nsteps;
  unsigned int g = 0;
  bool ok = n > 0;
  for (long long pos = 0; pos < total && ok; ++pos) {
    const unsigned int s = g % NSLOT;
    if (g >= NSLOT) ok = wait_bar(c, c.w_empty + 8 * s, ((g / NSLOT) - 1) & 1u);
    if (!ok) break;
    mbar_expect_tx(c.w_full + 8 * s, CHUNK_BYTES);
    bulk_g2s(c.sbase + RING_OFF + s * CHUNK_BYTES, base + (size_t)seq[pos % n] * (CHUNK_BYTES / 16), CHUNK_BYTES, c.w_full + 8 * s, pol);
    ++g;
  }
  if (!ok) {
    // give the copies still in flight time to land before the CTA can retire (bounded)
    for (unsigned int i = (g > NSLOT ? g - NSLOT : 0); i < g; ++i) {
      const uint32_t bar = c.w_full + 8 * (i % NSLOT);
      for (int tries = 0; tries < 20000 && !mbar_try_wait(bar, (i / NSLOT) & 1u); ++tries) __nanosleep(50);
    }
  }
}

// ---- activation loads (warp 9, one lane) ----------------------------------------------------------------------------------------
// Follows the same phase sequence as the MMA warps.  Phase j may read what other CTAs wrote once j grid barriers have
// been passed (thread 0 publishes the count); the loads of a phase are issued at once, as far as the four stages reach,
// and the rest as stages are handed back.
__device__ __forceinline__ void activation_producer_loop(Ctx& c) {
  const Params& p = *c.p;
  const uint64_t pol = policy_evict_last();
  unsigned int g = 0, att_n = 0;
  int phase = -1;
  bool ok = true;
  // Start of the next phase: wait until the grid barrier in front of it has completed (every CTA has arrived), tell the
  // MMA warps, and order the copies that follow behind the other CTAs' writes.
  auto begin_phase = [&]() {
    ++phase;
    if (!ok || phase == 0) return;
    const unsigned int target = (unsigned int)phase * (unsigned int)p.G;
    const uint64_t t0 = globaltimer_ns();
    unsigned int spins = 0, v;
    // one load in flight per CTA: sampling the counter more often (three relaxed loads in flight and an acquire fence
    // behind the one that saw the target) made every barrier 0.5 us slower, the L2 slice that holds the counter being
    // shared with the 148 arrivals
    for (;;) {
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p.bar_ctr) : "memory");
      if (v >= target) break;
      if ((++spins & 63u) == 0) {
        if (poll_abort(c)) { ok = false; return; }
        if (globaltimer_ns() - t0 > VLA_WAIT_LIMIT_NS) { raise_timeout(c); ok = false; return; }
      }
    }
    __threadfence_block();
    *c.go_count = phase;
    XP_LOG(c, 3400, 300, 1);
    // the rows were written to global memory through the generic proxy, the copies below read them through the async
    // one: a proxy fence restricted to global memory (the unrestricted one costs 0.25 us more per phase)
    asm volatile("fence.proxy.async.global;" ::: "memory");
  };
  // one stage = four 64-wide K blocks of MAX_ROWS rows from row0 on (rows past the tensor are filled with zeros), one copy
  auto stages = [&](const CUtensorMap* tm, int n_stages, int row0) {
    for (int st = 0; st < n_stages && ok; ++st) {
      const unsigned int s = g & 3u;
      if (g >= 4) ok = wait_bar(c, c.a_empty + 8 * s, ((g >> 2) - 1) & 1u);
      if (!ok) return;
      mbar_expect_tx(c.a_full + 8 * s, STAGE_BYTES);
      tma_load_3d(c.sbase + s * STAGE_BYTES, tm, c.a_full + 8 * s, 0, row0, st * 4, pol);
      ++g;
      XP_LOG(c, 3400, 300, 2);
    }
  };
  const int nq = qkv_tile_count(c.cta, p.G);
  const bool owner = c.cta < N_OWNERS;
  const int n_items = p.att_nrb * p.att_ks;
  for (int step = 0; step < p.nsteps && ok; ++step) {
    begin_phase();                                  // action in-projection: the MMA threads load its 50 x 32 tile themselves
    if (!p.pi05) {                                  // action MLP
      begin_phase();
      if (owner) stages(&p.tm_act, 4, 0);
    }
    for (int l = 0; l < p.nl && ok; ++l) {
      c.fine = p.trace != nullptr && c.cta == 0 && step == 0 && l == 1;
      begin_phase();                                // QKV
      if (nq > 0) stages(&p.tm_xb, 4, 0);
      begin_phase();                                // attention: K, V and Q tiles of this CTA's work item
      if (c.cta < n_items && ok) {
        // the four stages of the QKV phase have been handed back by every warp before the barrier just passed
        const int rb = c.cta / p.att_ks, sp = c.cta - rb * p.att_ks;
        const int row_k = l * p.T + sp * p.att_kps;
        const uint32_t kv_tile = (uint32_t)p.att_kps * 128;
        mbar_expect_tx(c.att_full, 4 * 4096 + 4 * kv_tile);
        mbar_expect_tx(c.att_full_v, 4 * kv_tile);
        tma_load_3d(c.sbase + ATT_Q_OFF, &p.tm_q, c.att_full, 0, rb * ATT_ROWS, 0, pol);   // the four 64-dim blocks in one copy each
        tma_load_3d(c.sbase, &p.tm_k, c.att_full, 0, row_k, 0, pol);
        tma_load_3d(c.sbase + ATT_V_OFF, &p.tm_v, c.att_full_v, 0, row_k, 0, pol);         // needed only after the softmax
        ++att_n;
      }
      begin_phase();                                // merge: reads global memory directly
      begin_phase();                                // attention-out projection
      if (owner) stages(&p.tm_attn, 8, 0);
      begin_phase();                                // GeGLU
      if (owner) stages(&p.tm_xb, 4, 0);
      begin_phase();                                // down projection
      if (owner) stages(&p.tm_hidden, 16, 0);
    }
    begin_phase();                                  // out-projection + Euler update
    if (c.cta < 4) stages(&p.tm_xb, 4, p.pi05 ? 0 : 1);
  }
  if (ok) begin_phase();                            // the barrier behind the last phase: release the MMA warps
  if (!ok) {
    // bounded wait for copies still in flight
    for (unsigned int i = (g > 4 ? g - 4 : 0); i < g; ++i)
      for (int tries = 0; tries < 20000 && !mbar_try_wait(c.a_full + 8 * (i & 3u), (i >> 2) & 1u); ++tries) __nanosleep(50);
    if (att_n > 0)
      for (int tries = 0; tries < 20000 && !(mbar_try_wait(c.att_full, (att_n - 1) & 1u) && mbar_try_wait(c.att_full_v, (att_n - 1) & 1u)); ++tries) __nanosleep(50);
  }
}

// ---- the kernel ----------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(THREADS, 1) expert_persistent_kernel(const __grid_constant__ Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw & 1023u)) & 1023u;
  Ctx c;
  c.p = &p;
  c.sbase = raw + pad;
  c.sptr = smem_raw + pad;
  uint8_t* persist = c.sptr + PERSIST_OFF;
  c.w_full = c.sbase + PERSIST_OFF;
  c.w_empty = c.w_full + 8 * NSLOT;
  c.a_full = c.w_empty + 8 * NSLOT;
  c.a_empty = c.a_full + 8 * N_ASTAGE;
  c.att_full = c.a_empty + 8 * N_ASTAGE;
  c.att_full_v = c.att_full + 8;
  c.umma_bar = c.att_full_v + 8;
  c.umma_n = 0;
  c.go_count = reinterpret_cast<volatile int*>(persist + 256);
  c.s_abort = reinterpret_cast<volatile int*>(persist + 260);
  c.fs = reinterpret_cast<float*>(persist + 512);
  c.xs = reinterpret_cast<float*>(persist + 768);        // 64 x 8 floats = 2 KB
  c.sttok = reinterpret_cast<float*>(persist + 2816);
  c.rope = reinterpret_cast<float2*>(persist + 3072);    // 3 x 4 x 64 float2 = 6 KB
  c.pk = 0;
  c.chunk_g = 0;
  c.a_g = 0;
  c.att_n = 0;
  c.bar_epoch = 0;
  c.fine = false;
  c.nmark = 0;
  c.cta = blockIdx.x;
  c.tid = threadIdx.x;
  c.warp = threadIdx.x >> 5;
  c.lane = threadIdx.x & 31;
  c.valid_len = p.valid_len_ptr ? *p.valid_len_ptr : p.P;
  c.pos_base = p.pi05 ? (p.pos_base_ptr ? *p.pos_base_ptr : p.P - 1) : p.P;
  if (threadIdx.x == 0) {
    for (int s = 0; s < NSLOT; ++s) {
      mbar_init(c.w_full + 8 * s, 1);
      mbar_init(c.w_empty + 8 * s, 8);
    }
    for (int s = 0; s < N_ASTAGE; ++s) {
      mbar_init(c.a_full + 8 * s, 1);
      mbar_init(c.a_empty + 8 * s, 8);
    }
    mbar_init(c.att_full, 1);
    mbar_init(c.att_full_v, 1);
    for (int j = 0; j < 8; ++j) mbar_init(c.umma_bar + 8 * j, 1);
    *c.go_count = 0;
    *c.s_abort = 0;
    mbar_fence_init();
  }
  for (int i = threadIdx.x; i < 64 * 8; i += THREADS) c.xs[i] = 0.f;
  for (int i = threadIdx.x; i < 3 * 4 * 64; i += THREADS) {   // rotary factors of this CTA's QKV feature pairs (V: identity)
    const int r = i & 63, pair = (i >> 6) & 3, t = i >> 8;
    const int n = 8 * (c.cta + t * p.G) + 2 * pair;
    float2 v = make_float2(1.f, 0.f);
    if (n < 2304 && r < p.S) {
      const int pos = c.pos_base + r, fi = (n & 255) >> 1;
      v = make_float2(p.rope_cos[pos * 128 + fi], p.rope_sin[pos * 128 + fi]);
    }
    c.rope[i] = v;
  }
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(persist + 264);   // behind the mbarriers (25 x 8 bytes) and the two words at 256
  if (c.warp == 0) tmem_alloc(smem_u32(tmem_slot), 64);   // GeGLU accumulator
  if (threadIdx.x == 32 * 9) {
    tma_prefetch_desc(&p.tm_xb); tma_prefetch_desc(&p.tm_attn); tma_prefetch_desc(&p.tm_hidden);
    tma_prefetch_desc(&p.tm_q); tma_prefetch_desc(&p.tm_k); tma_prefetch_desc(&p.tm_v);
    if (!p.pi05) tma_prefetch_desc(&p.tm_act);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  c.tmem = *tmem_slot;

  if (c.warp == 8) {
    if (c.lane == 0) weight_producer_loop(c);
    __syncwarp();
  } else if (c.warp == 9) {
    if (c.lane == 0) activation_producer_loop(c);
    __syncwarp();
  } else {
    bool ok = true;   // false once the kernel is being aborted
    if (!p.pi05 && c.cta < N_OWNERS && c.tid < 8) {   // state token features of this CTA (pi0_infer.py:1166-1171)
      const int n = 8 * c.cta + c.tid;
      float acc = p.b_state[n];
      for (int k = 0; k < 32; ++k) acc += __bfloat162float(p.state[k]) * __bfloat162float(p.w_state[(size_t)n * 64 + k]);
      c.sttok[c.tid] = acc;
    }
    // The kernel's schedule as one loop over phases, so that the code of every phase exists once (the kernel is larger
    // than the instruction cache; every copy costs fetch time).  Per Euler step: in-projection, (Pi0) action MLP, per
    // layer QKV, attention, merge, attention-out, GeGLU, down; then the out-projection.  A grid barrier follows every
    // phase.  What a phase function returns (a wait of this warp gave up) is not used for control flow: the abort word,
    // read behind a CTA barrier and so the same in every MMA thread, is.
    enum { K_IN, K_MLP, K_QKV, K_ATT, K_MRG, K_O, K_GEGLU, K_DOWN, K_OUT };
    const int head = p.pi05 ? 1 : 2;
    const int per_step = head + 6 * p.nl + 1;
#pragma unroll 1
    for (int ph = 0; ph < p.nsteps * per_step && ok; ++ph) {
      const int step = ph / per_step, r = ph - step * per_step;
      int kind, l = 0;
      if (r < head) kind = r == 0 ? K_IN : K_MLP;
      else if (r == per_step - 1) kind = K_OUT;
      else { l = (r - head) / 6; kind = K_QKV + (r - head) - 6 * l; }
      const size_t sl = (size_t)step * p.nl + l;
      c.fine = p.trace != nullptr && c.cta == 0 && step == 0 && l == 1 && kind >= K_QKV && kind <= K_DOWN;
      switch (kind) {
        case K_IN: phase_in_proj(c, step); break;
        case K_MLP: phase_action_mlp(c); break;
        case K_QKV: phase_qkv(c, step, l); break;
        case K_ATT: phase_attention(c, l); break;
        case K_MRG: phase_attention_merge(c); break;
        case K_O:
        case K_DOWN: {
          const bool o = kind == K_O;
          const float* gate = nullptr;
          const float* next_scale = nullptr;
          if (p.pi05) {
            gate = (o ? p.style_attn : p.style_ffn) + sl * 3072 + 2048;
            next_scale = o ? p.style_ffn + sl * 3072
                           : ((l + 1 < p.nl) ? p.style_attn + (sl + 1) * 3072 : p.style_fin + (size_t)step * 3072);
          }
          phase_resid(c, o ? 2048 : 4096, gate, next_scale, !o && l + 1 == p.nl);
          break;
        }
        case K_GEGLU: phase_geglu(c, step, l); break;
        default: phase_out(c, step); break;
      }
      ok = grid_barrier(c, ph);
    }
    c.fine = false;
    if (!ok) *c.s_abort = 1;
  }
  tc_fence_before();
  __syncthreads();
  if (c.warp == 0) tmem_dealloc(c.tmem, 64);
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
//   j = 5..12  MLP gate / up: K eighth j - 5 of all eight tiles as a tcgen05 operand (see below)
//   j = 13..16 MLP down tile c, K quarter j - 13
__global__ void pack_layer_kernel(const bf16* __restrict__ w_qkv, const bf16* __restrict__ w_o, const bf16* __restrict__ w_gate,
                                  const bf16* __restrict__ w_up, const bf16* __restrict__ w_down, int layer, int chunks_per_cta,
                                  bf16* __restrict__ stream) {
  const int j = blockIdx.x, cta = blockIdx.y, G = gridDim.y;
  bf16* dst = stream + ((size_t)cta * chunks_per_cta + (size_t)layer * CH_PER_LAYER + j) * (CHUNK_BYTES / 2);
  if (j >= 5 && j < 13) {
    // MLP gate/up: chunk j - 5 holds K eighth j - 5 (128 K = two 64-wide K blocks) of this CTA's 32 hidden features as
    // the B operand of the tcgen05 MMAs: [K block (2)][row (64)][128 B], row = 16 pair + (gate 0..7 | up 8..15), the
    // 16-byte chunks of a row permuted by the 128-byte swizzle (logical chunk c of row r at c ^ (r & 7)).
    if (cta >= N_OWNERS) return;
    const int k8 = j - 5;
    for (int e = threadIdx.x; e < CHUNK_BYTES / 2; e += blockDim.x) {
      const int kb = e >> 12, row = (e >> 6) & 63, pc = (e >> 3) & 7, w8 = e & 7;   // physical 16-byte chunk pc of the row
      const int ch = pc ^ (row & 7);                                             // logical chunk stored there
      const int k = 128 * k8 + 64 * kb + 8 * ch + w8;
      const int pair = row >> 4, up = (row >> 3) & 1;
      const int n = 32 * cta + 8 * pair + (row & 7);
      dst[e] = (up ? w_up : w_gate)[(size_t)n * 1024 + k];
    }
    return;
  }
  const bf16* src;
  int Kp, n0, k0;
  if (j < 3) {
    const int tile = cta + j * G;
    if (tile >= 320) return;
    src = w_qkv; Kp = 1024; n0 = 8 * tile; k0 = 0;
  } else {
    if (cta >= N_OWNERS) return;
    if (j < 5) { src = w_o; Kp = 2048; n0 = 8 * cta; k0 = 1024 * (j - 3); }
    else { src = w_down; Kp = 4096; n0 = 8 * cta; k0 = 1024 * (j - 13); }
  }
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
