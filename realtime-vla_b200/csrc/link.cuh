// Multi-view latency mode: the projected image tokens of the camera views travel from the GPUs that ran the SigLIP
// towers into the GPU that runs the prefix, inside the captured graphs, with plain peer stores over NVLink.
//
// The reference is single-GPU (its vision_encoder, pi0_infer.py:598-646, runs the views as one batch), so this exchange
// has no counterpart there; it replaces the NCCL gather between two graph launches.
//
//   tower (one per view, any GPU)                         trunk (prefix + action expert)
//   push_kernel, last node of the vision stage:           wait_kernel, first node of the prefix stage:
//     wait until the trunk has consumed forward e - 2       wait until flag[v] >= e for every view
//     copy the (256, 2048) fp32 tile into slot e & 1        copy slot e & 1 of every view into the residual stream
//       of the trunk's staging area (peer stores)           release ack[v] = e into every tower's mailbox (peer store)
//     release flag[view] = e (peer store)
//
// e counts forwards; both sides keep their own counter in their mailbox and advance it once per launch, so the graphs
// need no per-launch argument.  Two staging slots and the ack word bound how far a tower can run ahead of the trunk:
// nothing is overwritten before it has been consumed.  Every wait is bounded and raises the status word.
// No TMA, no multicast and no library kernel touches peer memory: 16-byte st.global and 4-byte release stores only.
#pragma once
#include "common.cuh"

namespace lk {

constexpr int TILE_FLOATS = 256 * 2048;   // projected tokens of one view (fp32 residual-stream rows)
constexpr int MAX_VIEWS = 16;
// trunk mailbox (words): [0, 64) flag per view, [64] forward counter, [65] blocks done, [66] failures, [67] views;
// byte 512: unsigned* ack[MAX_VIEWS] (where to acknowledge view v); byte 1024: staging [2][n_views][TILE_FLOATS]
constexpr int TRUNK_EPOCH = 64, TRUNK_DONE = 65, TRUNK_FAIL = 66, TRUNK_VIEWS = 67;   // [67]: number of views, set at creation
constexpr int TRUNK_ACK_OFF = 512, TRUNK_STAGING_OFF = 1024;
// tower mailbox (words): [0] ack written by the trunk, [16] forward counter, [17] blocks done, [18] failures
constexpr int TOWER_ACK = 0, TOWER_EPOCH = 16, TOWER_DONE = 17, TOWER_FAIL = 18;
constexpr int TOWER_BOX_BYTES = 256;

__device__ __forceinline__ bool wait_ge_sys(const unsigned int* p, unsigned int target, int* status) {
  const uint64_t t0 = globaltimer_ns();
  for (;;) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    if ((int)(v - target) >= 0) return true;
    if (globaltimer_ns() - t0 > VLA_WAIT_LIMIT_NS) {
      if (status) atomicOr(status, VLA_ST_WAIT_TIMEOUT);
      return false;
    }
    __nanosleep(200);
  }
}
__device__ __forceinline__ void store_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// true in the block that retires last (every other block's writes are then visible to it)
__device__ __forceinline__ bool last_block_done(unsigned int* counter) {
  __threadfence_system();
  const unsigned int prev = atomicAdd(counter, 1u);
  if (prev + 1 != gridDim.x) return false;
  *counter = 0;
  __threadfence_system();
  return true;
}

// tile: this tower's projected tokens [256, 2048] fp32; staging / flags: the trunk's mailbox (peer or local memory)
__global__ void __launch_bounds__(256) push_kernel(const float4* __restrict__ tile, float4* staging, unsigned int* flags,
                                                   unsigned int* box, int view, int n_views, int* status) {
  __shared__ int s_ok;
  const unsigned int e = box[TOWER_EPOCH] + 1;   // changes only when the last block retires: the same in every block
  if (threadIdx.x == 0) s_ok = (e <= 2u) ? 1 : (int)wait_ge_sys(box + TOWER_ACK, e - 2u, status);
  __syncthreads();
  if (s_ok) {
    float4* dst = staging + ((size_t)(e & 1u) * n_views + view) * (TILE_FLOATS / 4);
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < TILE_FLOATS / 4; i += gridDim.x * blockDim.x) dst[i] = tile[i];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (!s_ok) atomicOr(box + TOWER_FAIL, 1u);
    if (last_block_done(box + TOWER_DONE)) {
      const bool ok = box[TOWER_FAIL] == 0;
      box[TOWER_FAIL] = 0;
      if (ok) store_release_sys(flags + view, e);   // not published after a timeout: the trunk then gives up as well
      box[TOWER_EPOCH] = e;
    }
  }
}

// box: the trunk's mailbox (local); x: the prefix residual stream, view v occupies rows 256 v ..
__global__ void __launch_bounds__(256) wait_kernel(float4* __restrict__ x, unsigned int* box, int n_views, int* status) {
  __shared__ int s_ok;
  const unsigned int e = box[TRUNK_EPOCH] + 1;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if ((int)threadIdx.x < n_views && !wait_ge_sys(box + threadIdx.x, e, status)) s_ok = 0;
  __syncthreads();
  if (s_ok) {
    const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const uint8_t*>(box) + TRUNK_STAGING_OFF) +
                        (size_t)(e & 1u) * n_views * (TILE_FLOATS / 4);
    const int n = n_views * (TILE_FLOATS / 4);
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) x[i] = __ldcg(src + i);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (!s_ok) atomicOr(box + TRUNK_FAIL, 1u);
    if (last_block_done(box + TRUNK_DONE)) {
      box[TRUNK_FAIL] = 0;
      unsigned int** ack = reinterpret_cast<unsigned int**>(reinterpret_cast<uint8_t*>(box) + TRUNK_ACK_OFF);
      // the slot has been copied out (or the launch gave up): the towers may reuse it two forwards from now
      for (int v = 0; v < n_views; ++v)
        if (ack[v]) store_release_sys(ack[v], e);
      box[TRUNK_EPOCH] = e;
    }
  }
}

}  // namespace lk
