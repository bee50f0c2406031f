// Softmax attention with head dim 256 on the 5th-generation tensor cores (tcgen05 + TMEM), for the prefix
// and suffix attention of the Gemma stacks (one shared K/V head: the 8 query heads of a token are 8 query rows).
//
// One CTA = 128 query rows (TMEM lanes) against 128-key chunks:
//     S[128 x 128]  = Q[128 x 256] . K_chunk^T          tcgen05.mma, A = Q tile, B = K rows (both K-major)
//     P             = exp2(S*scale - rowmax)            one thread per query row, straight from TMEM
//     O[128 x 256] += P[128 x 128] . V_chunk            tcgen05.mma, A = P (bf16, written to shared memory in the
//                                                       128B-swizzled K-major layout), B = rows of V^T
// V is read from a transposed cache V^T[256][keys] so that both MMAs take plain K-major operands.  With more
// than one chunk the running maximum is kept per row and the O accumulator is rescaled in TMEM.  The keys can
// also be split over the CTAs of a cluster (grid.x); partial (O, max, sum) are merged in fixed order through an
// L2-resident scratch, as in the mma.sync kernel.  Roles: warp 0 = TMA producer, warp 1 = MMA issuer and
// TMEM owner, warps 2..9 = softmax / epilogue: two threads per query row, each owning one 64-key half of the
// chunk (= one P tile) and one 128-column half of O; they exchange only the row maximum.  The softmax is
// latency-bound (one warp per scheduler), hence two warps per TMEM lane quarter and branch-free masking.
// All mbarrier waits are bounded.
//
// Visibility of key j for query row i: see attention.cuh (same rule, same parameters).
#pragma once
#include <type_traits>
#include "common.cuh"

struct AttnTcParams {
  CUtensorMap tmQ;    // Q  [n_q rows, 256], box 64 x 128
  CUtensorMap tmK;    // K  [key rows, 256], box 64 x 128
  CUtensorMap tmVt;   // V^T [256 rows, keys], box 64 keys x 256
  bf16* o;            // [n_q, ldo]
  int ldo;
  int n_q, n_keys;
  int prefix_alloc, valid_prefix;
  const int* valid_prefix_ptr;
  int restrict_rows;
  float scale_log2e;
  int ksplit;
  float* scratch;     // [group][row block][rank][260 columns][128 rows] fp32 when ksplit > 1
  int* status;
  // groups = independent observations along grid.z: group g uses query/output rows g*q_group_rows.., key rows
  // g*k_group_rows.. and rows g*256.. of the transposed value tensor; masks and lengths are the same for all
  int q_group_rows, k_group_rows;
};

struct AttnTcCfg {
  static constexpr int Q_BYTES = 128 * 256 * 2;     // 4 tiles [128 x 64]
  static constexpr int K_BYTES = 128 * 256 * 2;     // 4 tiles [128 keys x 64]
  static constexpr int V_BYTES = 256 * 128 * 2;     // 2 tiles [256 d x 64 keys]
  static constexpr int P_BYTES = 128 * 128 * 2;     // 2 tiles [128 rows x 64 keys]
  static constexpr int BAR_BYTES = 128 + 2 * 128 * 4;   // barriers + TMEM slot, then the row-maximum exchange [2][128]
  static constexpr int SMEM_BYTES = Q_BYTES + K_BYTES + V_BYTES + P_BYTES + BAR_BYTES + 1024;
  static constexpr int SCOLS = 260;                 // scratch columns per split: 256 outputs, max, sum half 0, sum half 1, pad
  static constexpr int THREADS = 320;
  static constexpr int TMEM_COLS = 512;             // S: columns [0,128), O: columns [128,384)
};

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]),
        "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]),
        "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint64_t attn_desc_sw128(uint32_t smem_addr) {
  return (uint64_t)((smem_addr & 0x3FFFF) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void named_barrier_sync(int id, int n_threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n_threads) : "memory");
}

__device__ __forceinline__ uint64_t low_bits64(int n) { return n >= 64 ? ~0ull : ((1ull << n) - 1ull); }

__global__ void __launch_bounds__(AttnTcCfg::THREADS, 1) attention_tc_kernel(const __grid_constant__ AttnTcParams p) {
  using C = AttnTcCfg;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  const uint32_t sQ = raw_addr + pad;
  const uint32_t sK = sQ + C::Q_BYTES;
  const uint32_t sV = sK + C::K_BYTES;
  const uint32_t sP = sV + C::V_BYTES;
  uint8_t* sP_ptr = smem + C::Q_BYTES + C::K_BYTES + C::V_BYTES;
  const uint32_t bars = sP + C::P_BYTES;
  const uint32_t q_full = bars, k_full = bars + 8, v_full = bars + 16, s_full = bars + 24, p_ready = bars + 32,
                 o_done = bars + 40;
  uint8_t* bar_ptr = smem + C::Q_BYTES + C::K_BYTES + C::V_BYTES + C::P_BYTES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_ptr + 64);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile float* xchg = reinterpret_cast<volatile float*>(bar_ptr + 128);   // [2 halves][128 rows]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  KTRACE(20);
  const int rank = blockIdx.x, ksplit = p.ksplit;
  const int row0 = blockIdx.y * 128;
  const int q_base = blockIdx.z * p.q_group_rows, k_base = blockIdx.z * p.k_group_rows, vt_base = blockIdx.z * 256;
  const int n_chunks_total = (p.n_keys + 127) / 128;
  const int ch_begin = (int)(((long long)rank * n_chunks_total) / ksplit);
  const int ch_end = (int)(((long long)(rank + 1) * n_chunks_total) / ksplit);
  const int n_chunks = ch_end - ch_begin;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(k_full, 1);
    mbar_init(v_full, 1);
    mbar_init(s_full, 1);
    mbar_init(p_ready, 256);
    mbar_init(o_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&p.tmQ);
    tma_prefetch_desc(&p.tmK);
    tma_prefetch_desc(&p.tmVt);
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base, tmem_O = tmem_base + 128;

  pdl_trigger();
  pdl_wait();
  KTRACE(21);

  if (warp == 0) {
    if (lane == 0 && n_chunks > 0) {
      const uint64_t pol = policy_evict_last();
      mbar_expect_tx(q_full, C::Q_BYTES);
      for (int kb = 0; kb < 4; ++kb) tma_load_2d(sQ + kb * 16384, &p.tmQ, q_full, kb * 64, q_base + row0, pol);
      for (int c = 0; c < n_chunks; ++c) {
        const int key0 = (ch_begin + c) * 128;
        // K buffer is free once the S MMAs of the previous chunk have completed
        if (c > 0 && !mbar_wait(s_full, (uint32_t)(c - 1) & 1u, abort_flag)) break;
        mbar_expect_tx(k_full, C::K_BYTES);
        for (int kb = 0; kb < 4; ++kb) tma_load_2d(sK + kb * 16384, &p.tmK, k_full, kb * 64, k_base + key0, pol);
        // V buffer is free once the PV MMAs of the previous chunk have completed
        if (c > 0 && !mbar_wait(o_done, (uint32_t)(c - 1) & 1u, abort_flag)) break;
        mbar_expect_tx(v_full, C::V_BYTES);
        for (int kb = 0; kb < 2; ++kb) tma_load_2d(sV + kb * 32768, &p.tmVt, v_full, key0 + kb * 64, vt_base, pol);
        KTRACE_B(23, 0, p.ksplit - 1);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0 && n_chunks > 0) {
      const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((128u >> 3) << 17) | (8u << 24);
      const uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | ((256u >> 3) << 17) | (8u << 24);
      bool ok = mbar_wait(q_full, 0, abort_flag);
      for (int c = 0; c < n_chunks && ok; ++c) {
        const uint32_t ph = (uint32_t)c & 1u;
        ok = mbar_wait(k_full, ph, abort_flag);
        if (!ok) break;
        tc_fence_after();
        KTRACE_B(24, 32, p.ksplit - 1);
#pragma unroll
        for (int kb = 0; kb < 4; ++kb) {
          const uint64_t da = attn_desc_sw128(sQ + kb * 16384), db = attn_desc_sw128(sK + kb * 16384);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) umma_bf16(tmem_S, da + 2 * kk, db + 2 * kk, idesc_s, (kb | kk) != 0);
        }
        umma_commit(s_full);
        ok = mbar_wait(p_ready, ph, abort_flag) && mbar_wait(v_full, ph, abort_flag);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kb = 0; kb < 2; ++kb) {
          const uint64_t da = attn_desc_sw128(sP + kb * 16384), db = attn_desc_sw128(sV + kb * 32768);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) umma_bf16(tmem_O, da + 2 * kk, db + 2 * kk, idesc_o, (c | kb | kk) != 0);
        }
        umma_commit(o_done);
      }
    }
    __syncwarp();
  }

  // ---------------- softmax / epilogue: two threads per query row ----------------
  const bool is_sm = warp >= 2;
  const int q = warp & 3;                 // TMEM lane quarter
  const int half = (warp - 2) >> 2;       // which 64 keys of a chunk / which 128 columns of O this thread owns
  const int r = q * 32 + lane;            // row within the block = TMEM lane
  const int i = row0 + r;                 // global query row
  const uint32_t lane_off = (uint32_t)(q * 32) << 16;
  float m_run = -1e30f, l_run = 0.f;      // l_run: sum over this thread's keys only
  const bool warp_live = row0 + q * 32 < p.n_q;   // warp-uniform: false when all 32 rows lie beyond n_q
  bool ok = true;
  if (is_sm) {
    const int valid_prefix = p.valid_prefix_ptr ? min(max(*p.valid_prefix_ptr, 0), p.prefix_alloc) : p.valid_prefix;
    // key j is visible to this row iff  j < lim1  ||  lo2 <= j <= hi2
    const int lim1 = min(valid_prefix, p.n_keys);
    const int lo2 = p.prefix_alloc;
    const int hi2 = min(p.n_keys - 1, i >= p.restrict_rows ? p.n_keys - 1 : p.prefix_alloc);
    // Both warps of a lane quarter run every iteration and meet at one named barrier per chunk even after a
    // wait has timed out (ok == false), so that a timeout in one of them can never strand the other.
    for (int c = 0; c < n_chunks; ++c) {
      const uint32_t ph = (uint32_t)c & 1u;
      ok = ok && __all_sync(0xffffffffu, mbar_wait(s_full, ph, abort_flag));   // warp-uniform: TMEM loads are collective
      tc_fence_after();
      KTRACE_B(25, 64, p.ksplit - 1);
      const int key0 = (ch_begin + c) * 128 + half * 64;
      // Visibility of this thread's 64 keys as a bit mask.  Most chunks are entirely visible; the one or two
      // that straddle the prefix/suffix boundaries test one bit per key; a half chunk without a visible key
      // (beyond the last key, or a warp whose 32 rows all lie beyond n_q) only clears its half of P.  The
      // mode is warp-uniform because the TMEM loads below are warp-collective.
      uint64_t vmask;
      {
        const int n1 = min(max(lim1 - key0, 0), 64);
        const int a2 = min(max(lo2 - key0, 0), 64), b2 = min(max(hi2 + 1 - key0, 0), 64);
        vmask = low_bits64(n1) | (b2 > a2 ? (low_bits64(b2) & ~low_bits64(a2)) : 0ull);
        if (!warp_live) vmask = 0ull;
      }
      const bool all_vis = __all_sync(0xffffffffu, vmask == ~0ull);
      const bool none_vis = __all_sync(0xffffffffu, vmask == 0ull);
      // pass 1: masked, scaled logits of this thread's 64 keys -> maximum
      float m_loc = -1e30f;
      if (ok && !none_vis) {
#pragma unroll
        for (int c0 = 0; c0 < 64; c0 += 32) {
          uint32_t v[32];
          tmem_ld32(tmem_S + lane_off + half * 64 + c0, v);
          tmem_ld_wait();
          float mx[4] = {-3.0e38f, -3.0e38f, -3.0e38f, -3.0e38f};
          if (all_vis) {
#pragma unroll
            for (int j = 0; j < 32; ++j) mx[j & 3] = fmaxf(mx[j & 3], __uint_as_float(v[j]));
          } else {
            const uint32_t w = (uint32_t)(vmask >> c0);
#pragma unroll
            for (int j = 0; j < 32; ++j) mx[j & 3] = fmaxf(mx[j & 3], (w >> j) & 1u ? __uint_as_float(v[j]) : -3.0e38f);
          }
          // the scale is positive, so it commutes with the maximum
          m_loc = fmaxf(m_loc, fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * p.scale_log2e);
        }
        m_loc = fmaxf(m_loc, -1e30f);
      }
      xchg[half * 128 + r] = m_loc;
      named_barrier_sync(1 + q, 64);      // the two warps of this lane quarter
      if (!ok) continue;
      const float m_new = fmaxf(m_run, fmaxf(m_loc, xchg[(half ^ 1) * 128 + r]));
      const float alpha = ex2_approx(m_run - m_new);
      // pass 2: probabilities -> bf16 P tile `half` in the swizzled K-major layout, row sum
      float ls[4] = {0.f, 0.f, 0.f, 0.f};
      uint8_t* tile = sP_ptr + half * 16384 + r * 128;
      if (none_vis) {
#pragma unroll
        for (int cidx = 0; cidx < 8; ++cidx) *reinterpret_cast<uint4*>(tile + (cidx << 4)) = make_uint4(0u, 0u, 0u, 0u);
      } else {
        auto pass2 = [&](auto av) {
#pragma unroll
          for (int c0 = 0; c0 < 64; c0 += 32) {
            uint32_t v[32];
            tmem_ld32(tmem_S + lane_off + half * 64 + c0, v);
            tmem_ld_wait();
            const uint32_t w = (uint32_t)(vmask >> c0);
            uint32_t pk[16];
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              float e[2];
#pragma unroll
              for (int u = 0; u < 2; ++u) {
                const float ex = ex2_approx(fmaf(__uint_as_float(v[j + u]), p.scale_log2e, -m_new));
                e[u] = (decltype(av)::value || ((w >> (j + u)) & 1u)) ? ex : 0.f;
              }
              const __nv_bfloat162 h = __floats2bfloat162_rn(e[0], e[1]);
              // the row sum uses the rounded probabilities, i.e. exactly what the PV product sees
              ls[(j >> 1) & 3] += __bfloat162float(h.x) + __bfloat162float(h.y);
              pk[j >> 1] = *reinterpret_cast<const uint32_t*>(&h);
            }
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const int cidx = (c0 >> 3) + g;   // 16-byte chunk of the 128-byte row
              *reinterpret_cast<uint4*>(tile + ((cidx ^ (r & 7)) << 4)) = make_uint4(pk[4 * g], pk[4 * g + 1], pk[4 * g + 2], pk[4 * g + 3]);
            }
          }
        };
        if (all_vis) pass2(std::true_type{}); else pass2(std::false_type{});
      }
      l_run = l_run * alpha + ((ls[0] + ls[1]) + (ls[2] + ls[3]));
      m_run = m_new;
      if (c > 0 && warp_live) {   // rescale this thread's half of the running output (the previous PV MMAs completed before s_full)
#pragma unroll 1
        for (int c0 = 0; c0 < 128; c0 += 32) {
          uint32_t v[32];
          tmem_ld32(tmem_O + lane_off + half * 128 + c0, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * alpha);
          tmem_st32(tmem_O + lane_off + half * 128 + c0, v);
        }
        tmem_st_wait();
      }
      KTRACE_B(26, 64, p.ksplit - 1);
      fence_proxy_async_smem();   // P (generic-proxy stores) must be visible to the tensor core's async reads
      tc_fence_before();
      mbar_arrive(p_ready);
    }
    if (ok && n_chunks > 0) {
      ok = __all_sync(0xffffffffu, mbar_wait(o_done, (uint32_t)(n_chunks - 1) & 1u, abort_flag));
      tc_fence_after();
      KTRACE_B(27, 64, p.ksplit - 1);
    }
  }

  if (ksplit == 1) {
    // tcgen05.ld is warp-collective (.sync.aligned): every lane of the warp executes it, rows beyond n_q only
    // skip the global store (a warp may straddle n_q: 408 suffix rows = 3 blocks + 24 rows)
    if (is_sm) {
      xchg[half * 128 + r] = l_run;
      named_barrier_sync(1 + q, 64);
      const float l_tot = l_run + xchg[(half ^ 1) * 128 + r];
      if (ok && n_chunks > 0) {
        const bool row_ok = i < p.n_q;
        const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
        bf16* orow = p.o + (size_t)(q_base + (row_ok ? i : 0)) * p.ldo + half * 128;
#pragma unroll 1
        for (int c0 = 0; c0 < 128; c0 += 32) {
          uint32_t v[32];
          tmem_ld32(tmem_O + lane_off + half * 128 + c0, v);
          tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint4 w;
              w.x = pack_bf16(__uint_as_float(v[j]) * inv, __uint_as_float(v[j + 1]) * inv);
              w.y = pack_bf16(__uint_as_float(v[j + 2]) * inv, __uint_as_float(v[j + 3]) * inv);
              w.z = pack_bf16(__uint_as_float(v[j + 4]) * inv, __uint_as_float(v[j + 5]) * inv);
              w.w = pack_bf16(__uint_as_float(v[j + 6]) * inv, __uint_as_float(v[j + 7]) * inv);
              *reinterpret_cast<uint4*>(orow + c0 + j) = w;
            }
          }
          __syncwarp();
        }
      }
    }
  } else {
    // ---- merge the key splits through the L2-resident scratch, fixed rank order ----
    // layout per split: [260 columns][128 rows]: 256 outputs, max, row sum of half 0, row sum of half 1
    float* cl = p.scratch + (size_t)(blockIdx.z * gridDim.y + blockIdx.y) * ksplit * C::SCOLS * 128;
    if (is_sm) {
      float* mine = cl + (size_t)rank * C::SCOLS * 128;
      const bool live = ok && n_chunks > 0;
      if (warp_live) {   // rows beyond n_q are never read back
        if (live) {
#pragma unroll 1
          for (int c0 = 0; c0 < 128; c0 += 32) {
            uint32_t v[32];
            tmem_ld32(tmem_O + lane_off + half * 128 + c0, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) __stcg(mine + (half * 128 + c0 + j) * 128 + r, __uint_as_float(v[j]));
          }
        }
        // a split without chunks contributes (max = -1e30, sums = 0) and gets zero weight
        if (half == 0) __stcg(mine + 256 * 128 + r, live ? m_run : -1e30f);
        __stcg(mine + (257 + half) * 128 + r, live ? l_run : 0.f);
      }
    }
    __syncwarp();
    KTRACE_B(28, 64, p.ksplit - 1);
    cluster_sync_all();
    KTRACE_B(29, 64, p.ksplit - 1);
    if (is_sm) {
      // This CTA finishes the head-dim slice [rank * width, (rank + 1) * width) of every live row.  One item =
      // one row x 8 consecutive outputs; items are spread over all 256 threads (the TMEM lane rule no longer
      // binds a row to a warp here) and every load of an item is issued before the first use, so the merge
      // costs one L2 round trip.
      const int rows_here = min(128, p.n_q - row0);
      const int rstride = rows_here <= 32 ? 32 : (rows_here <= 64 ? 64 : 128);
      const int width = 256 / ksplit;
      const int n_items = rstride * (width >> 3);
      for (int item = (int)threadIdx.x - 64; item < n_items; item += 256) {
        const int rr = item & (rstride - 1);
        const int d0 = rank * width + (item / rstride) * 8;
        if (rr >= rows_here) continue;
        float mr[8], lr[8], a[8][8];
#pragma unroll
        for (int s2 = 0; s2 < 8; ++s2) {
          mr[s2] = -1e30f;
          lr[s2] = 0.f;
          if (s2 < ksplit) {
            const float* src = cl + (size_t)s2 * C::SCOLS * 128;
            mr[s2] = __ldcg(src + 256 * 128 + rr);
            lr[s2] = __ldcg(src + 257 * 128 + rr) + __ldcg(src + 258 * 128 + rr);
          }
#pragma unroll
          for (int e = 0; e < 8; ++e) a[s2][e] = (s2 < ksplit) ? __ldcg(cl + ((size_t)s2 * C::SCOLS + d0 + e) * 128 + rr) : 0.f;
        }
        float m_tot = -1e30f, l_tot = 0.f, w[8];
#pragma unroll
        for (int s2 = 0; s2 < 8; ++s2) m_tot = fmaxf(m_tot, mr[s2]);
#pragma unroll
        for (int s2 = 0; s2 < 8; ++s2) {
          w[s2] = lr[s2] > 0.f ? ex2_approx(mr[s2] - m_tot) : 0.f;
          l_tot += lr[s2] * w[s2];
        }
        const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          o[e] = 0.f;
#pragma unroll
          for (int s2 = 0; s2 < 8; ++s2) o[e] += a[s2][e] * w[s2];   // fixed rank order
        }
        uint4 wv;
        wv.x = pack_bf16(o[0] * inv, o[1] * inv);
        wv.y = pack_bf16(o[2] * inv, o[3] * inv);
        wv.z = pack_bf16(o[4] * inv, o[5] * inv);
        wv.w = pack_bf16(o[6] * inv, o[7] * inv);
        *reinterpret_cast<uint4*>(p.o + (size_t)(q_base + row0 + rr) * p.ldo + d0) = wv;
      }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0 && p.status) atomicOr(p.status, VLA_ST_WAIT_TIMEOUT);
    for (int k = 0; k < 32; ++k) __nanosleep(1000);
  }
  if (warp == 1) tmem_dealloc(tmem_base, C::TMEM_COLS);
  KTRACE(22);
}
