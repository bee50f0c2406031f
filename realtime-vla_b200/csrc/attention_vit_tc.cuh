// SigLIP attention on the tcgen05 tensor cores: 16 heads of dim 72 over the 256 patch tokens of one camera view,
// no mask (AttnMultiKey of the reference, pi0_infer.py:588-596: per-view scaled-dot-product attention on the
// [Q | K | V] rows of the QKV GEMM, scale 72^-0.5).
//
// One CTA = one (view, head, 128-query block); grid (2, 16, views).  A head slice is 72 bf16 = 144 bytes inside
// a 6 912-byte row, which no 128-byte-swizzled TMA box can fetch without dragging in the neighbouring head, so
// the operands are brought in with 16-byte vector loads and written into the canonical K-major, 128-byte-swizzled
// shared-memory layout by the threads themselves:
//   Q  [128 rows][80 dims]  two K blocks (64 dims, then 8 real dims + 8 zeros)        A of S = Q K^T
//   K  [256 keys][80 dims]  same                                                        B of S
//   V^T[80 dims ][256 keys] four K blocks of 64 keys, rows 72..79 zero                  B of O = P V
//   P  [128 rows][256 keys] four K blocks, written by the softmax threads               A of O
// S (128 x 256, fp32) and O (128 x 80) live in TMEM.  All 256 keys fit one S tile, so the softmax is a single
// pass pair (maximum, then exponentials) by two threads per query row (128 keys each), with no running rescale.
// Every wait on an mbarrier is bounded; a wait that runs out raises the status word instead of hanging.
#pragma once
#include "attention_tc.cuh"

#ifdef VLA_TRACE
#define VIT_TRACE(slot) do { if (p.trace && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 128) p.trace[slot] = clock64(); } while (0)
#else
#define VIT_TRACE(slot) do {} while (0)
#endif

struct VitAttnTcParams {
  const bf16* qkv;   // [views * 256, 3456] = [Q | K | V], each 16 heads x 72
  bf16* o;           // [views * 256, 1152]
  float scale_log2e; // 72^-0.5 * log2(e)
  int* status;
  long long* trace;  // development timeline (-DVLA_TRACE), normally null
};

struct VitAttnTcCfg {
  static constexpr int Q_BYTES = 2 * 128 * 128;    // two K blocks of [128 rows x 128 B]
  static constexpr int K_BYTES = 2 * 256 * 128;    // two K blocks of [256 keys x 128 B]
  static constexpr int V_BYTES = 4 * 80 * 128;     // four K blocks of [80 dims x 128 B (64 keys)]
  static constexpr int P_BYTES = 4 * 128 * 128;    // four K blocks of [128 rows x 128 B (64 keys)]
  static constexpr int BAR_BYTES = 128 + 2 * 128 * 4;
  static constexpr int SMEM_BYTES = Q_BYTES + K_BYTES + V_BYTES + P_BYTES + BAR_BYTES + 1024;
  static constexpr int THREADS = 256;
  static constexpr int TMEM_COLS = 512;            // S: columns [0,256), O: columns [256,336)
};

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}

__global__ void __launch_bounds__(VitAttnTcCfg::THREADS, 1) vit_attention_tc_kernel(const VitAttnTcParams p) {
  using C = VitAttnTcCfg;
  extern __shared__ uint8_t vit_smem_raw[];
  const uint32_t raw_addr = smem_u32(vit_smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = vit_smem_raw + pad;
  const uint32_t sQ = raw_addr + pad, sK = sQ + C::Q_BYTES, sV = sK + C::K_BYTES, sP = sV + C::V_BYTES;
  uint8_t* pQ = smem;
  uint8_t* pK = pQ + C::Q_BYTES;
  uint8_t* pV = pK + C::K_BYTES;
  uint8_t* pP = pV + C::V_BYTES;
  uint8_t* bar_ptr = pP + C::P_BYTES;
  const uint32_t bars = sP + C::P_BYTES;
  const uint32_t s_done = bars, o_done = bars + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_ptr + 64);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile float* xchg = reinterpret_cast<volatile float*>(bar_ptr + 128);   // [2 halves][128 rows]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row0 = blockIdx.x * 128, head = blockIdx.y, view = blockIdx.z;
  VIT_TRACE(0);

  if (tid == 0) {
    mbar_init(s_done, 1);
    mbar_init(o_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_S = *tmem_slot, tmem_O = tmem_S + 256;

  pdl_trigger();
  pdl_wait();
  VIT_TRACE(1);

  // ---------------- operands into the swizzled K-major layout ----------------
  // a row of a [rows x 128 B] K block holds eight 16-byte chunks; chunk c of row r sits at r*128 + ((c ^ (r & 7)) << 4)
  const bf16* base = p.qkv + (size_t)view * 256 * 3456 + head * 72;
  const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
  // All global loads of a thread are issued before the first shared-memory store, so that they share one L2
  // round trip: Q 5, K 10, V 9 vectors of 16 bytes per thread.
  uint4 qv[5], kv[10], vv[9];
#pragma unroll
  for (int j = 0; j < 5; ++j) {      // Q: 128 rows x 10 chunks (9 of data + 1 of zeros completing the last 16 dims)
    const int i = tid + j * C::THREADS, r = i / 10, c = i - r * 10;
    qv[j] = c < 9 ? *reinterpret_cast<const uint4*>(base + (size_t)(row0 + r) * 3456 + c * 8) : zero4;
  }
#pragma unroll
  for (int j = 0; j < 10; ++j) {     // K: 256 keys x 10 chunks
    const int i = tid + j * C::THREADS, r = i / 10, c = i - r * 10;
    kv[j] = c < 9 ? *reinterpret_cast<const uint4*>(base + 1152 + (size_t)r * 3456 + c * 8) : zero4;
  }
#pragma unroll
  for (int j = 0; j < 9; ++j)        // V: key = tid, chunk j (consecutive threads take consecutive keys)
    vv[j] = *reinterpret_cast<const uint4*>(base + 2304 + (size_t)tid * 3456 + j * 8);
  VIT_TRACE(2);
#pragma unroll
  for (int j = 0; j < 5; ++j) {
    const int i = tid + j * C::THREADS, r = i / 10, c = i - r * 10, kb = c >> 3, cc = c & 7;
    *reinterpret_cast<uint4*>(pQ + kb * 16384 + r * 128 + ((cc ^ (r & 7)) << 4)) = qv[j];
  }
#pragma unroll
  for (int j = 0; j < 10; ++j) {
    const int i = tid + j * C::THREADS, r = i / 10, c = i - r * 10, kb = c >> 3, cc = c & 7;
    *reinterpret_cast<uint4*>(pK + kb * 32768 + r * 128 + ((cc ^ (r & 7)) << 4)) = kv[j];
  }
  // V^T: element (d, key) of K block key/64 at d*128 + (((key%64)/8 ^ (d & 7)) << 4) + (key % 8) * 2; rows 72..79 zero
  {
    const int i = tid;                 // 8 zero rows x 4 K blocks x 8 chunks = 256 vectors
    const int d = 72 + (i >> 5), kb = (i >> 3) & 3, cc = i & 7;
    *reinterpret_cast<uint4*>(pV + kb * 10240 + d * 128 + (cc << 4)) = zero4;
    const int key = tid, kc = (key & 63) >> 3;
    uint8_t* blk = pV + (key >> 6) * 10240 + (key & 7) * 2;
#pragma unroll
    for (int c = 0; c < 9; ++c) {
      const bf16* e = reinterpret_cast<const bf16*>(&vv[c]);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int d2 = c * 8 + j;
        *reinterpret_cast<bf16*>(blk + d2 * 128 + ((kc ^ (d2 & 7)) << 4)) = e[j];
      }
    }
  }
  VIT_TRACE(3);
  fence_proxy_async_smem();   // generic-proxy stores -> visible to the tensor core's async-proxy reads
  __syncthreads();
  VIT_TRACE(4);

  // ---------------- S = Q K^T ----------------
  if (warp == 0 && lane == 0) {
    tc_fence_after();
    const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((256u >> 3) << 17) | (8u << 24);
    // dims 0..63: four k16 steps of K block 0; dims 64..79: one step of K block 1
#pragma unroll
    for (int kk = 0; kk < 4; ++kk)
      umma_bf16(tmem_S, attn_desc_sw128(sQ) + 2 * kk, attn_desc_sw128(sK) + 2 * kk, idesc_s, kk != 0);
    umma_bf16(tmem_S, attn_desc_sw128(sQ + 16384), attn_desc_sw128(sK + 32768), idesc_s, 1u);
    umma_commit(s_done);
  }
  __syncwarp();

  // ---------------- softmax: two threads per query row, 128 keys each ----------------
  const int q = warp & 3, half = warp >> 2;
  const int r = q * 32 + lane;
  const uint32_t lane_off = (uint32_t)(q * 32) << 16;
  bool ok = __all_sync(0xffffffffu, mbar_wait(s_done, 0, abort_flag));   // TMEM loads are warp-collective
  tc_fence_after();
  VIT_TRACE(5);
  // the 128 logits of this thread stay in registers between the two passes
  uint32_t sv[128];
  float m_loc = -1e30f;
  if (ok) {
#pragma unroll
    for (int c0 = 0; c0 < 128; c0 += 32) tmem_ld32(tmem_S + lane_off + half * 128 + c0, sv + c0);
    tmem_ld_wait();
    float mx[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) mx[j] = -3.0e38f;
#pragma unroll
    for (int j = 0; j < 128; ++j) mx[j & 7] = fmaxf(mx[j & 7], __uint_as_float(sv[j]));
    m_loc = fmaxf(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])), fmaxf(fmaxf(mx[4], mx[5]), fmaxf(mx[6], mx[7]))) * p.scale_log2e;
  }
  xchg[half * 128 + r] = m_loc;
  named_barrier_sync(1 + q, 64);      // the two warps of this lane quarter
  const float m_row = fmaxf(m_loc, xchg[(half ^ 1) * 128 + r]);
  named_barrier_sync(1 + q, 64);      // both have read the maxima before the sums reuse the slots
  float l_loc = 0.f;
  if (ok) {
#pragma unroll
    for (int c0 = 0; c0 < 128; c0 += 32) {
      uint32_t pk[16];
      float ls[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < 32; j += 2) {
        const float e0 = ex2_approx(fmaf(__uint_as_float(sv[c0 + j]), p.scale_log2e, -m_row));
        const float e1 = ex2_approx(fmaf(__uint_as_float(sv[c0 + j + 1]), p.scale_log2e, -m_row));
        const __nv_bfloat162 h = __floats2bfloat162_rn(e0, e1);
        ls[(j >> 1) & 3] += __bfloat162float(h.x) + __bfloat162float(h.y);   // sum of what the P V product sees
        pk[j >> 1] = *reinterpret_cast<const uint32_t*>(&h);
      }
      l_loc += (ls[0] + ls[1]) + (ls[2] + ls[3]);
      const int key0 = half * 128 + c0;                 // 32 keys = four 16-byte chunks of K block key0 / 64
      uint8_t* tile = pP + (key0 >> 6) * 16384 + r * 128;
      const int cbase = (key0 & 63) >> 3;
#pragma unroll
      for (int g = 0; g < 4; ++g)
        *reinterpret_cast<uint4*>(tile + (((cbase + g) ^ (r & 7)) << 4)) = make_uint4(pk[4 * g], pk[4 * g + 1], pk[4 * g + 2], pk[4 * g + 3]);
    }
  }
  VIT_TRACE(6);
  xchg[half * 128 + r] = l_loc;
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();             // P complete (and the row sums exchanged) before the MMA is issued
  const float l_tot = l_loc + xchg[(half ^ 1) * 128 + r];

  // ---------------- O = P V ----------------
  if (warp == 0 && lane == 0 && !*abort_flag) {
    tc_fence_after();
    const uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | ((80u >> 3) << 17) | (8u << 24);
#pragma unroll
    for (int kb = 0; kb < 4; ++kb) {
      const uint64_t da = attn_desc_sw128(sP + kb * 16384), db = attn_desc_sw128(sV + kb * 10240);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) umma_bf16(tmem_O, da + 2 * kk, db + 2 * kk, idesc_o, (kb | kk) != 0);
    }
    umma_commit(o_done);
  }
  __syncwarp();
  ok = ok && __all_sync(0xffffffffu, mbar_wait(o_done, 0, abort_flag));
  tc_fence_after();
  VIT_TRACE(7);
  if (ok) {
    // half 0 stores dims 0..31 and 64..71, half 1 dims 32..63 (80 accumulator columns, the last 8 are padding)
    const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
    bf16* orow = p.o + ((size_t)view * 256 + row0 + r) * 1152 + head * 72;
    uint32_t v[32], w[16];
    tmem_ld32(tmem_O + lane_off + half * 32, v);
    if (half == 0) tmem_ld16(tmem_O + lane_off + 64, w);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
      uint4 u;
      u.x = pack_bf16(__uint_as_float(v[j]) * inv, __uint_as_float(v[j + 1]) * inv);
      u.y = pack_bf16(__uint_as_float(v[j + 2]) * inv, __uint_as_float(v[j + 3]) * inv);
      u.z = pack_bf16(__uint_as_float(v[j + 4]) * inv, __uint_as_float(v[j + 5]) * inv);
      u.w = pack_bf16(__uint_as_float(v[j + 6]) * inv, __uint_as_float(v[j + 7]) * inv);
      *reinterpret_cast<uint4*>(orow + half * 32 + j) = u;
    }
    if (half == 0) {
      uint4 u;
      u.x = pack_bf16(__uint_as_float(w[0]) * inv, __uint_as_float(w[1]) * inv);
      u.y = pack_bf16(__uint_as_float(w[2]) * inv, __uint_as_float(w[3]) * inv);
      u.z = pack_bf16(__uint_as_float(w[4]) * inv, __uint_as_float(w[5]) * inv);
      u.w = pack_bf16(__uint_as_float(w[6]) * inv, __uint_as_float(w[7]) * inv);
      *reinterpret_cast<uint4*>(orow + 64) = u;
    }
  }

  // ---------------- teardown ----------------
  VIT_TRACE(8);
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (tid == 0 && p.status) atomicOr(p.status, VLA_ST_WAIT_TIMEOUT);
  }
  if (warp == 1) tmem_dealloc(tmem_S, C::TMEM_COLS);
}
