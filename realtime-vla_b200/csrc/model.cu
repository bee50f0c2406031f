// Host side of libvla_b200.so: weight repacking, buffer layout, the launch plan of one Pi0 / Pi05 forward,
// its capture into one CUDA graph, and the C ABI declared in include/vla_b200.h.
//
// Data layout in HBM (one observation; a batch multiplies the token counts):
//   weights      bf16, K-major [features_pad128, K_pad64] per layer (transposed once from the checkpoint's [K, N])
//   biases, LayerNorm scale/shift, position embedding, adaRMS styles, RoPE tables   fp32
//   residual streams vision_x [256*nv,1152], encoder_x [P,2048], decoder_x [S,1024], noise [C,32]   fp32
//   GEMM operands (normalised activations, attention outputs, MLP hidden)   bf16 row-major
//   K/V cache    bf16 [layer][observation][P + S][256]; prefix rows first, the S suffix rows rewritten each step
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <functional>
#include <map>
#include <mutex>
#include <set>
#include <string>
#include <vector>

#include "../../include/vla_b200.h"
#include "attention.cuh"
#include "attention_tc.cuh"
#include "attention_vit_tc.cuh"
#include "elementwise.cuh"
#include "expert_persistent.cuh"
#include "gemm_sm100.cuh"
#include "link.cuh"
#include "preprocess.cuh"

namespace {

thread_local std::string g_last_error;

// The persistent action-expert kernel serves eligible handles by default when true; flags bit 5 selects it
// explicitly, bit 4 refuses it.
constexpr bool XP_DEFAULT_ON = true;

// ---------------------------------------------------------------------------------------------------
// driver entry point for tensor-map encoding (no link-time dependency on libcuda)
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// bf16 [rows, K] row-major with row pitch ld (elements): box = 64 (K) x box_rows, 128-byte swizzle.
bool make_tmap(CUtensorMap* tm, const void* base, long long K, long long rows, long long ld, int box_rows,
               std::string* err) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) { *err = "cuTensorMapEncodeTiled entry point not found"; return false; }
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[256];
    snprintf(buf, sizeof buf, "cuTensorMapEncodeTiled failed (%d) K=%lld rows=%lld ld=%lld box_rows=%d base=%p", (int)r, K,
             rows, ld, box_rows, base);
    *err = buf;
    return false;
  }
  return true;
}

// The same operand as a 3-D map (64 elements, rows, K / 64 blocks): one copy of box 64 x box_rows x box_blocks lands as
// [block][row][128 B], i.e. box_blocks consecutive 64-wide K blocks of the same rows (rows past the tensor read as zeros).
bool make_tmap3(CUtensorMap* tm, const void* base, long long K, long long rows, long long ld, int box_rows, int box_blocks,
                std::string* err) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) { *err = "cuTensorMapEncodeTiled entry point not found"; return false; }
  cuuint64_t dims[3] = {64u, (cuuint64_t)rows, (cuuint64_t)(K / 64)};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, 128u};
  cuuint32_t box[3] = {64u, (cuuint32_t)box_rows, (cuuint32_t)box_blocks};
  cuuint32_t estr[3] = {1u, 1u, 1u};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[256];
    snprintf(buf, sizeof buf, "cuTensorMapEncodeTiled (3-D) failed (%d) K=%lld rows=%lld ld=%lld box_rows=%d base=%p", (int)r, K,
             rows, ld, box_rows, base);
    *err = buf;
    return false;
  }
  return true;
}

// output tile map for TMA stores: [rows, cols] row-major with pitch ld (elements), box 32 x 32, no swizzle
bool make_out_tmap(CUtensorMap* tm, const void* base, bool f32, long long cols, long long rows, long long ld, std::string* err) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) { *err = "cuTensorMapEncodeTiled entry point not found"; return false; }
  const int esz = f32 ? 4 : 2;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * esz};
  cuuint32_t box[2] = {32u, 32u};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = fn(tm, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
                  strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[200];
    snprintf(buf, sizeof buf, "cuTensorMapEncodeTiled (output) failed (%d) cols=%lld rows=%lld ld=%lld", (int)r, cols, rows, ld);
    *err = buf;
    return false;
  }
  return true;
}

// ---------------------------------------------------------------------------------------------------
// generic launch with optional cluster dimension and programmatic dependent launch
template <typename... KArgs, typename... Args>
cudaError_t launch_ex(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, int cluster_x, bool pdl,
                      Args&&... args) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof cfg);
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attrs[2];
  int n = 0;
  if (cluster_x > 1) {
    attrs[n].id = cudaLaunchAttributeClusterDimension;
    attrs[n].val.clusterDim.x = cluster_x;
    attrs[n].val.clusterDim.y = 1;
    attrs[n].val.clusterDim.z = 1;
    ++n;
  }
  if (pdl) {
    attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// The dynamic shared-memory opt-in of a kernel applies to the CURRENT device only, so it is remembered per
// (device, kernel): a process may hold handles on several GPUs.
cudaError_t ensure_smem_attr(const void* func, int bytes) {
  static std::mutex mu;
  static std::set<std::pair<int, const void*>> done;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  std::lock_guard<std::mutex> lock(mu);
  if (done.count({dev, func})) return cudaSuccess;
  e = cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) done.insert({dev, func});
  return e;
}

// ---------------------------------------------------------------------------------------------------
// GEMM launch plan
struct GemmOp {
  GemmParams p;
  int bn;
  bool dual;
  dim3 grid;
};

// Every tile shape exists as a split-K (cluster) variant.
bool can_split(int, bool) { return true; }

// Scratch floats a GEMM launch needs for its split-K partial tiles (0 without split).
size_t gemm_scratch_floats(int bn, bool dual, dim3 grid, int cg2 = 0) {
  if (grid.x <= (cg2 ? 2u : 1u)) return 0;
  return (size_t)grid.x * grid.y * grid.z * 128 * bn * (dual ? 2 : 1);
}

int pick_split(int units, int k_blocks, int sm_count) {
  int split = 1;
  // Split while all CTAs still fit the SMs in one wave (clusters of 8 fit ~16 at a time on the 8 GPCs).
  while (split < 8 && units * split * 2 <= sm_count && split * 2 <= k_blocks) split *= 2;
  return split;
}

// Token tile and K split for a GEMM of `tokens` rows over feat_tiles x k_blocks weight tiles.
// Up to 128 tokens there is one token tile and the split follows pick_split.  Above that a small cost
// model (in SM cycles) chooses between 128- and 256-token tiles and K splits of 1, 2, 4, 8:
//   per CTA and 64-wide K block: TMA brings 16 KB per weight tile + 128 B per token row at ~64 B/clk (the
//   per-SM L2 read rate, measured 59-62 B/clk), the MMAs take 2*bn clk per accumulator, whichever is longer;
//   + epilogue ~22 clk per token column and accumulator (two warps per lane quarter), + ~5000 clk for the
//   split-K exchange; x the number of waves over the SMs.
// A single-weight GEMM may also pair two feature tiles in one CTA (m256: 256 features x bn tokens, two
// accumulators sharing the activation tile like the gate/up pair): 32 KB + 128 B per token per K block for twice
// the MMA work, which lifts 256-token tiles from TMA-bound (96 B/clk) to balanced (64 B/clk) at the price of half
// as many CTAs and a twice larger split-K exchange.  m256_mode: 0 = let the model choose, 1 = force, -1 = never.
// A third shape, cg2, runs neighbouring feature tiles as tcgen05 CTA pairs that share the activation tile, each CTA
// loading half of it (16 KB + 64 B per token per K block and CTA): same CTA count and exchange as the plain shape.
// cg2_mode: 0 = let the model choose, 1 = force, -1 = never.
// Tokens per CTA along grid.y for `tokens` rows in tiles of at most b: the tiles are evened out (788 tokens = 4 x 224
// rather than 3 x 256 + 20), and a launch that fits the SMs in one wave with room to spare takes more, smaller tiles
// (multiples of 32) until the wave is full: the K loop of a CTA is bound by its MMAs (2 clk per token and 16-wide K
// step) or by the bytes it pulls from L2, both of which shrink with the tile (SigLIP QKV at 768 tokens: 27 feature
// tiles x 3 token tiles of 256 = 81 CTAs become 27 x 5 tiles of 160 = 135 CTAs).  ctas_per_tok_tile = CTAs per
// token tile (feature tiles x K split).
int even_tok_tile(int tokens, int b, int ctas_per_tok_tile, int resident, bool fill_wave) {
  int tok_tile = b;
  int n_tiles = (tokens + b - 1) / b;
  if (tokens > b) tok_tile = std::min(b, ((tokens + n_tiles - 1) / n_tiles + 31) / 32 * 32);
  if (fill_wave && tokens >= 192 && ctas_per_tok_tile * n_tiles <= resident) {
    n_tiles = std::min(std::max(n_tiles, resident / ctas_per_tok_tile), (tokens + 31) / 32);
    tok_tile = std::min(tok_tile, ((tokens + n_tiles - 1) / n_tiles + 31) / 32 * 32);
  }
  return tok_tile;
}

// qkv: the launch has the QKV epilogue, whose split-K form (rotary table loads and cache-row arithmetic per owned column,
// scattered stores of the transposed values) measured 5 us slower than the unsplit tile-store form at 256 tokens.
void pick_tiling(int tokens, int feat_tiles, int k_blocks, bool dual, int sm_count, int* bn, int* split, int* m256,
                 int m256_mode = 0, int* cg2 = nullptr, int cg2_mode = 0, bool qkv = false) {
  *m256 = 0;
  if (cg2) *cg2 = 0;
  if (tokens <= 128 && m256_mode <= 0) {
    *bn = tokens <= 64 ? 64 : 128;
    *split = pick_split(feat_tiles, k_blocks, sm_count);
    return;
  }
  double best = 1e30;
  *bn = 256;
  *split = 1;
  // up to 256 tokens a 128-token tile always measured at least as fast as one 256-token tile (more CTAs, a
  // cheaper split-K exchange); dual-accumulator GEMMs keep 256 (their main loop is MMA-bound only there)
  const int b_max = (tokens <= 256 && !dual) ? 128 : 256;
  for (int shape = 0; shape <= 2; ++shape) {   // 0 plain, 1 paired feature tiles in one CTA, 2 CTA pairs
    const int pair = shape == 1, two = shape == 2;
    if (pair && (dual || m256_mode < 0 || feat_tiles < 2)) continue;
    if (!pair && m256_mode > 0 && !dual && feat_tiles >= 2) continue;
    if (two && (!cg2 || cg2_mode < 0 || feat_tiles < 2)) continue;
    if (!two && cg2 && cg2_mode > 0 && feat_tiles >= 2) continue;
    const int accs = (dual || pair) ? 2 : 1;
    const int ftiles = pair ? (feat_tiles + 1) / 2 : (two ? (feat_tiles + 1) / 2 * 2 : feat_tiles);
    for (int b = 128; b <= ((pair || two) ? 256 : b_max); b *= 2) {
      if (two && dual && b != 256) continue;              // the dual CTA-pair kernel exists for 256-token tiles only
      for (int s = 1; s <= (two ? 4 : 8); s *= 2) {       // a cluster holds at most 8 CTAs
        if (s > 1 && (k_blocks / s < 8)) continue;          // keep K slices long enough to amortise the exchange
        if (two && dual && s > 1) continue;
        const int tok_tiles = (tokens + b - 1) / b;
        const long long ctas = (long long)ftiles * tok_tiles * s;
        if (s > 1 && (size_t)ctas * 128 * b * accs > ((size_t)16 << 20)) continue;   // split-K scratch capacity (floats)
        // measured: a paired tile only pays unsplit and over several waves (batched forwards: 788 x 16384 x 2048
        // took 72 us paired with K split 4 against 68 us unpaired, 17 024 tokens 870 us against 1 076 us)
        if (pair && m256_mode == 0 && (s > 1 || ctas < 2LL * sm_count)) continue;
        const int kb = (k_blocks + s - 1) / s;
        // (costing an unsplit launch with the smaller token tiles it ends up with, see even_tok_tile, chose unsplit
        // long-K launches that measure slower: SigLIP down projection at 512 tokens 25.6 against 18.6 us; configuration 3
        // 11.65 -> 12.18 ms.  The tile shape is therefore chosen for the coarse tiles and refined afterwards.)
        const double load = kb * (16384.0 * accs + (two ? 64.0 : 128.0) * b) / 64.0;
        const double mma = kb * 2.0 * b * accs;
        const double epi = 22.0 * (b / 2) * accs;
        // partial tile through L2 + cluster barrier; measured cheaper than twice the 128-token figure for a 4-way
        // split of 256-token tiles (SigLIP down projection at 768 tokens: 22.7 us against 25.9 us for 128 x 2)
        const double exch = s > 1 ? 5000.0 * (b == 256 ? (s == 4 ? 1.5 : 2.0) : 1.0) * accs + (qkv ? 8000.0 : 0.0) : 0.0;
        const double cta = (load > mma ? load : mma) + epi + exch;
        // clusters are scheduled whole within a GPC: 144 CTAs in clusters of 4 measured like two waves
        // (512 x 4304 x 1152: 29 us against 25 us for 72 CTAs), so 4- and 8-CTA clusters count 128 resident CTAs
        const int resident = s * (two ? 2 : 1) >= 4 ? 128 : sm_count;
        const double waves = (double)((ctas + resident - 1) / resident);
        const double cost = waves * cta;
        if (cost < best) { best = cost; *bn = b; *split = s; *m256 = pair; if (cg2) *cg2 = two; }
      }
    }
  }
}

template <int BN, bool DUAL, bool SPLITK, bool PAIR = false, bool CG2 = false>
cudaError_t launch_gemm_t(const GemmOp& op, cudaStream_t st, bool pdl) {
  using C = GemmCfg<BN, DUAL || PAIR, SPLITK, CG2>;
  static_assert(C::VALID, "tile shape leaves fewer than 3 pipeline stages");
  auto kern = gemm_sm100_kernel<BN, DUAL, SPLITK, PAIR, CG2>;
  if (cudaError_t e = ensure_smem_attr(reinterpret_cast<const void*>(kern), C::SMEM_BYTES); e != cudaSuccess) return e;
  return launch_ex(kern, op.grid, dim3(GEMM_THREADS), C::SMEM_BYTES, st, op.p.split * (CG2 ? 2 : 1), pdl, op.p);
}

cudaError_t launch_gemm(const GemmOp& op, cudaStream_t st, bool pdl) {
  const bool sk = op.p.split > 1;
  if (op.p.cg2) {    // CTA pairs (built for 128- and 256-token tiles; dual only unsplit at 256)
    if (op.dual) return launch_gemm_t<256, true, false, false, true>(op, st, pdl);
    if (op.bn == 128) return sk ? launch_gemm_t<128, false, true, false, true>(op, st, pdl) : launch_gemm_t<128, false, false, false, true>(op, st, pdl);
    return sk ? launch_gemm_t<256, false, true, false, true>(op, st, pdl) : launch_gemm_t<256, false, false, false, true>(op, st, pdl);
  }
  if (op.p.m256) {   // two feature tiles of one weight per CTA
    if (op.bn == 64) return sk ? launch_gemm_t<64, false, true, true>(op, st, pdl) : launch_gemm_t<64, false, false, true>(op, st, pdl);
    if (op.bn == 128) return sk ? launch_gemm_t<128, false, true, true>(op, st, pdl) : launch_gemm_t<128, false, false, true>(op, st, pdl);
    return sk ? launch_gemm_t<256, false, true, true>(op, st, pdl) : launch_gemm_t<256, false, false, true>(op, st, pdl);
  }
  if (op.bn == 64) {
    if (op.dual) return sk ? launch_gemm_t<64, true, true>(op, st, pdl) : launch_gemm_t<64, true, false>(op, st, pdl);
    return sk ? launch_gemm_t<64, false, true>(op, st, pdl) : launch_gemm_t<64, false, false>(op, st, pdl);
  }
  if (op.bn == 128) {
    if (op.dual) return sk ? launch_gemm_t<128, true, true>(op, st, pdl) : launch_gemm_t<128, true, false>(op, st, pdl);
    return sk ? launch_gemm_t<128, false, true>(op, st, pdl) : launch_gemm_t<128, false, false>(op, st, pdl);
  }
  if (op.dual) return sk ? launch_gemm_t<256, true, true>(op, st, pdl) : launch_gemm_t<256, true, false>(op, st, pdl);
  return sk ? launch_gemm_t<256, false, true>(op, st, pdl) : launch_gemm_t<256, false, false>(op, st, pdl);
}

// w / w2: repacked weights [n_feat_pad, Kp]; x: activations [tokens, K] with pitch ldx.
bool build_gemm(GemmOp* op, const bf16* w, const bf16* w2, int n_feat, int n_feat_pad, int Kp, const bf16* x, int tokens,
                int Kx, int ldx, const GemmEpi& epi, int* status, int sm_count, int force_bn, int force_split,
                std::string* err, int m256_mode = 0, int force_tok_tile = 0, int cg2_mode = 0, bool fill_wave = true) {
  memset(op, 0, sizeof *op);
  op->dual = w2 != nullptr;
  if (Kp % 64 || n_feat_pad % 128) { *err = "repacked weight must be padded to 128 features x 64 K"; return false; }
  int feat_tiles = n_feat_pad / 128;
  const int kb = Kp / 64;
  int bn, split, m256, cg2;
  pick_tiling(tokens, feat_tiles, kb, op->dual, sm_count, &bn, &split, &m256, m256_mode, &cg2, cg2_mode,
              epi.kind == EPI_QKV && epi.rows_per_obs >= tokens);
  if (force_bn > 0) {
    bn = force_bn;
    if (bn != 64 && bn != 128 && bn != 256) { *err = "token tile must be 64, 128 or 256"; return false; }
    m256 = (m256_mode > 0 && !op->dual && feat_tiles >= 2) ? 1 : 0;
    cg2 = (cg2_mode > 0 && feat_tiles >= 2) ? 1 : 0;
    split = can_split(bn, op->dual) ? pick_split((m256 ? (feat_tiles + 1) / 2 : feat_tiles) * ((tokens + bn - 1) / bn), kb, sm_count) : 1;
    if (cg2 && split > 4) split = 4;
  }
  if (force_split > 0) split = force_split;
  if (cg2) {
    if (m256) { *err = "a launch is either paired feature tiles or CTA pairs"; return false; }
    if (bn == 64 || (op->dual && (bn != 256 || split > 1)) || split > 4) {
      *err = "CTA pairs: 128- or 256-token tiles, K split <= 4; two weights only unsplit with 256-token tiles";
      return false;
    }
  }
  op->p.cg2 = cg2;
  if (m256) {
    op->dual = true;                       // two accumulators, both fed from `w`
    feat_tiles = (feat_tiles + 1) / 2;
  }
  op->p.m256 = m256;
  op->bn = bn;
  // Even out the token tiles and fill the wave (fill_wave = false keeps the coarse tiles: more CTAs also mean more
  // split-K scratch, which the allocation-free entry point takes from a fixed array).
  int tok_tile = even_tok_tile(tokens, bn, (cg2 ? 2 * ((feat_tiles + 1) / 2) : feat_tiles) * split,
                               split * (cg2 ? 2 : 1) >= 4 ? 128 : sm_count, fill_wave && !m256);
  if (force_tok_tile > 0) {
    if (force_tok_tile % 32 || force_tok_tile > bn) { *err = "token tile stride must be a multiple of 32 and <= bn"; return false; }
    tok_tile = force_tok_tile;
  }
  op->p.tok_tile = tok_tile;
  const int tok_tiles = (tokens + tok_tile - 1) / tok_tile;
  if (split > 1 && !can_split(bn, op->dual)) { *err = "this tile shape has no split-K variant"; return false; }
  if (split > 8 || split > kb || (split & (split - 1))) { *err = "split must be 1, 2, 4 or 8 and <= K/64"; return false; }
  if (!make_tmap(&op->p.tmA, w, Kp, n_feat_pad, Kp, 128, err)) return false;
  if (w2 && !make_tmap(&op->p.tmA2, w2, Kp, n_feat_pad, Kp, 128, err)) return false;
  if (!make_tmap(&op->p.tmB, x, Kx, tokens, ldx, cg2 ? tok_tile / 2 : tok_tile, err)) return false;
  op->p.n_feat = n_feat;
  op->p.n_tok = tokens;
  op->p.k_blocks = kb;
  op->p.split = split;
  // Large-token, unsplit launches write their output tiles through TMA where the epilogue is a plain tile
  // write: bf16 outputs, and fp32 residual outputs without row remapping or a bf16 mirror.
  op->p.out_mode = 0;
  if (split == 1 && tokens > 64) {
    if (epi.kind == EPI_BF16 && (epi.ld_out * 2) % 16 == 0 && ((uintptr_t)epi.out % 16) == 0) {
      if (!make_out_tmap(&op->p.tmOut, epi.out, false, n_feat, tokens, epi.ld_out, err)) return false;
      op->p.out_mode = 1;
    } else if (epi.kind == EPI_RESID && epi.out_rpo == 0 && epi.res_mod == 0 && !epi.mirror && (epi.ld_outf * 4) % 16 == 0 &&
               ((uintptr_t)epi.outf % 16) == 0 && (epi.res_in == nullptr || (epi.res_in == epi.outf && epi.ld_res == epi.ld_outf))) {
      if (!make_out_tmap(&op->p.tmOut, epi.outf, true, n_feat, tokens, epi.ld_outf, err)) return false;
      op->p.out_mode = epi.res_in ? 3 : 2;
    } else if (epi.kind == EPI_QKV && epi.rows_per_obs >= tokens) {
      if (!make_out_tmap(&op->p.tmOut, epi.q, false, 2048, tokens, 2048, err)) return false;
      if (!make_out_tmap(&op->p.tmOut2, epi.kc, false, 256, epi.kv_row_off + tokens, 256, err)) return false;
      if (!make_out_tmap(&op->p.tmOut3, epi.vc, false, 256, epi.kv_row_off + tokens, 256, err)) return false;
      op->p.out_mode = 4;
    }
  }
  op->p.status = status;
  op->p.epi = epi;
  op->grid = cg2 ? dim3(2 * split, tok_tiles, (feat_tiles + 1) / 2) : dim3(split, tok_tiles, feat_tiles);
  return true;
}

// ---------------------------------------------------------------------------------------------------
template <int HD>
cudaError_t launch_attn_t(const AttnParams& p, int groups, cudaStream_t st, bool pdl) {
  auto kern = attention_kernel<HD>;
  if (cudaError_t e = ensure_smem_attr(reinterpret_cast<const void*>(kern), AttnCfg<HD>::SMEM_BYTES); e != cudaSuccess) return e;
  dim3 grid(p.ksplit, (p.n_q + 63) / 64, groups);
  return launch_ex(kern, grid, dim3(128), AttnCfg<HD>::SMEM_BYTES, st, p.ksplit, pdl, p);
}
cudaError_t launch_attn(const AttnParams& p, int head_dim, int groups, cudaStream_t st, bool pdl) {
  return head_dim == 72 ? launch_attn_t<72>(p, groups, st, pdl) : launch_attn_t<256>(p, groups, st, pdl);
}
size_t attn_scratch_floats(const AttnParams& p, int head_dim, int groups) {
  if (p.ksplit <= 1) return 0;
  const int hdp = (head_dim + 15) / 16 * 16;
  return (size_t)groups * ((p.n_q + 63) / 64) * p.ksplit * 64 * (hdp + 4);
}
int pick_ksplit(int n_q, int n_keys, int groups, int sm_count) {
  const int ctas = ((n_q + 63) / 64) * groups, blocks = (n_keys + 63) / 64;
  int ks = 1;
  while (ks < 8 && ctas * ks * 2 <= (sm_count * 7) / 8 && ks * 2 <= blocks) ks *= 2;
  return ks;
}

// ---- tcgen05 attention (head dim 256, one group) ---------------------------------------------------
struct AttnTcOp {
  AttnTcParams p;
  dim3 grid;
};
int pick_ksplit_tc(int n_q, int n_keys, int sm_count, int groups = 1) {
  const int row_blocks = ((n_q + 127) / 128) * groups, chunks = (n_keys + 127) / 128;
  // From 16 query blocks on, one CTA per block over all keys measured at least as fast as a key split with its merge
  // through L2 (256 tokens x 8 heads: 14.6 against 18.7 us; 564: 22.8 against 24.8; 788: 28.9 against 28.4); the
  // suffix attention of the per-operator expert (4 query blocks, 7 chunks) keeps its split.
  if (row_blocks >= 16 && row_blocks <= 48) return 1;
  int ks = 1;
  while (ks < 8 && ks < chunks && row_blocks * ks * 2 <= sm_count) ks *= 2;
  return ks;
}
size_t attn_tc_scratch_floats(int n_q, int ksplit, int groups = 1) {
  return ksplit > 1 ? (size_t)groups * ((n_q + 127) / 128) * ksplit * 128 * AttnTcCfg::SCOLS : 0;
}
// q [n_q,256]; k [k_rows,256] (n_keys <= k_rows used); vt [256, vt_ld] transposed values
bool build_attn_tc(AttnTcOp* op, const bf16* q, const bf16* k, int k_rows, const bf16* vt, int vt_ld, bf16* o, int ldo, int n_q,
                   int n_keys, int prefix_alloc, int valid_prefix, const int* valid_ptr, int restrict_rows, float scale,
                   int ksplit, float* scratch, int* status, std::string* err, int groups = 1, int q_group_rows = 0) {
  memset(op, 0, sizeof *op);
  if (vt_ld % 8) { *err = "transposed value cache pitch must be a multiple of 8"; return false; }
  if (groups < 1) { *err = "attention needs at least one group"; return false; }
  if (groups == 1) q_group_rows = n_q;
  // groups: q [groups * q_group_rows, 256], k [groups * k_rows, 256], vt [groups * 256, vt_ld]
  if (!make_tmap(&op->p.tmQ, q, 256, (groups - 1) * q_group_rows + n_q, 256, 128, err)) return false;
  if (!make_tmap(&op->p.tmK, k, 256, groups * k_rows, 256, 128, err)) return false;
  if (!make_tmap(&op->p.tmVt, vt, vt_ld, groups * 256, vt_ld, 256, err)) return false;
  op->p.q_group_rows = q_group_rows; op->p.k_group_rows = k_rows;
  op->p.o = o; op->p.ldo = ldo; op->p.n_q = n_q; op->p.n_keys = n_keys;
  op->p.prefix_alloc = prefix_alloc; op->p.valid_prefix = valid_prefix; op->p.valid_prefix_ptr = valid_ptr;
  op->p.restrict_rows = restrict_rows; op->p.scale_log2e = scale * 1.4426950408889634f;
  op->p.ksplit = ksplit; op->p.scratch = scratch; op->p.status = status;
  op->grid = dim3(ksplit, (n_q + 127) / 128, groups);
  return true;
}
cudaError_t launch_attn_tc(const AttnTcOp& op, cudaStream_t st, bool pdl) {
  if (cudaError_t e = ensure_smem_attr(reinterpret_cast<const void*>(attention_tc_kernel), AttnTcCfg::SMEM_BYTES); e != cudaSuccess) return e;
  return launch_ex(attention_tc_kernel, op.grid, dim3(AttnTcCfg::THREADS), AttnTcCfg::SMEM_BYTES, st, op.p.ksplit, pdl, op.p);
}

// SigLIP attention of `views` camera views (16 heads x 72, 256 tokens each) on tcgen05
cudaError_t launch_vit_attn_tc(const VitAttnTcParams& p, int views, cudaStream_t st, bool pdl) {
  if (cudaError_t e = ensure_smem_attr(reinterpret_cast<const void*>(vit_attention_tc_kernel), VitAttnTcCfg::SMEM_BYTES); e != cudaSuccess) return e;
  return launch_ex(vit_attention_tc_kernel, dim3(2, 16, views), dim3(VitAttnTcCfg::THREADS), VitAttnTcCfg::SMEM_BYTES, st, 1, pdl, p);
}

cudaError_t launch_norm(const float* x, int ld_x, bf16* y, int ld_y, int rows, int D, int mode, const float* w,
                        const float* b, int in_rpo, int in_stride, int in_off, cudaStream_t st, bool pdl) {
  if (D == 1152) return launch_ex(norm_kernel<1152>, dim3(rows), dim3(128), 0, st, 1, pdl, x, ld_x, y, ld_y, mode, w, b, in_rpo, in_stride, in_off);
  if (D == 2048) return launch_ex(norm_kernel<2048>, dim3(rows), dim3(128), 0, st, 1, pdl, x, ld_x, y, ld_y, mode, w, b, in_rpo, in_stride, in_off);
  if (D == 1024) return launch_ex(norm_kernel<1024>, dim3(rows), dim3(128), 0, st, 1, pdl, x, ld_x, y, ld_y, mode, w, b, in_rpo, in_stride, in_off);
  return cudaErrorInvalidValue;
}

// ---------------------------------------------------------------------------------------------------
enum WKind { W_MATRIX, W_VECTOR, W_TIME_EMBEDS, W_PROMPT };
struct WSpec {
  WKind kind;
  bool layered;      // first dim = layer count
  int which_layers;  // 0 vit, 1 transformer, -1 none
  int K, N;          // matrix: [K,N]; vector: N
  int lead;          // non-layered vectors with a leading dim (time biases [10,1024], pos emb [256,1152])
};
struct WEntry {
  WSpec spec;
  int L, Kp, Np;
  bf16* w = nullptr;   // [L][Np][Kp]
  float* v = nullptr;  // [L or lead][N (padded to Np for bias of padded matrices)]
  bool loaded = false;
};

int round_up(int x, int m) { return (x + m - 1) / m * m; }

}  // namespace

// ===================================================================================================
struct vla_model {
  vla_config cfg;
  std::string err;
  bool pi05;
  int nv, C, L, B, P, S, T, nvl, nl, nsteps;
  int sm_count;
  bool use_pdl, use_graph;
  bool finalized = false;
  int valid_len;       // prefix tokens currently valid (views*256 + prompt rows)
  std::vector<void*> allocs;
  size_t bytes = 0;
  std::map<std::string, WEntry> W;
  std::map<std::string, std::pair<void*, size_t>> named;

  // I/O and activations
  bf16 *images, *state, *noise, *state_pad;
  float* noise_f32;
  bf16 *patches, *vision_xn, *vision_qkv, *vision_attn, *vision_hidden;
  float* vision_x;
  float* encoder_x;
  bf16 *encoder_xn, *encoder_q, *encoder_attn, *encoder_hidden;
  bf16 *kcache, *vcache, *vtcache;
  int T_pad;
  float *decoder_x, *state_tok;
  bf16* decoder_xb;      // bf16 copy of the un-normalised suffix stream (operand of the GEMMs with folded RMS norm)
  float* decoder_ssq;    // [32 slots][suffix tokens] partial sums of squares of that stream
  bf16 *decoder_xn, *decoder_q, *decoder_attn, *decoder_hidden, *decoder_act, *decoder_xfin;
  bf16* decoder_qkv = nullptr;   // batched forwards: bf16 output of the plain QKV GEMM [tokens, 2560]
  bf16* lang;
  float *rope_cos, *rope_sin;
  float *style_attn, *style_ffn, *style_fin;
  // folded adaRMS (Pi05 expert): shift rows as bf16 GEMM operands and shift @ W per (step, layer)
  bf16 *shift_attn_bf = nullptr, *shift_ffn_bf = nullptr;          // [layer][step][1024]
  float *sw_qkv = nullptr, *sw_gate = nullptr, *sw_up = nullptr;   // [step][layer][2560 | 4096 | 4096]
  bf16 *time_tmp, *time_emb;
  int *d_valid_len, *d_pos_base, *d_status;
  bf16* embed_table = nullptr;    // optional token embedding table [vocab, 2048] ('embedding_weight')
  int vocab = 0;
  int *d_ids = nullptr, *d_n_ids = nullptr;   // prompt token ids and their count (-1: prompt given as embeddings)
  int n_ids = -1;
  int* h_scalars = nullptr;       // pinned staging slots for the per-call scalars (64 x 3 ints)
  unsigned scalar_slot = 0;
  int* h_status = nullptr;        // pinned copy of the device status word read by vla_forward_host
  // pre/post-processing: resample tables per (input size, output size), frame staging that grows on demand
  struct ResampleTable { int ksize; int* bounds; int* kk; };
  std::map<std::pair<int, int>, ResampleTable> resample;
  uint8_t* pp_frame = nullptr;   // staged camera frame followed by the horizontally resampled picture
  size_t pp_frame_cap = 0;
  double* pp_vec = nullptr;      // [256] small float64 vectors (state, statistics)
  double* pp_out = nullptr;      // [chunk * 32] un-normalised actions
  float* gemm_scratch;            // split-K partial tiles of whichever GEMM is running (kernels never overlap)
  size_t gemm_scratch_cap = 0;    // floats
  float* attn_scratch;            // key-split partial outputs of whichever attention kernel is running
  size_t attn_scratch_cap = 0;
  // persistent action-expert kernel (single observation): per-CTA weight streams and its small exchange buffers
  bool use_xp = false;
  int xp_G = 0, xp_chunks = 0;
  uint4* xp_stream = nullptr;
  float *xp_part = nullptr, *xp_stat = nullptr, *xp_sw_fin = nullptr;
  unsigned int* xp_sync = nullptr;
  unsigned long long* xp_trace = nullptr;
  xp::Params xp_params;

  // multi-view latency mode over NVLink (link.cuh): this handle's mailbox and what it has opened of other processes
  uint8_t* link_box = nullptr;
  int link_views = 0;              // > 0: trunk mailbox for that many views; 0 with link_box set: tower mailbox
  bool link_connected = false;
  std::vector<void*> ipc_opened;

  struct Op { int stage; bool is_kernel; std::function<cudaError_t(cudaStream_t)> fn; };
  std::vector<Op> ops;
  int n_kernels = 0;
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t graph_exec = nullptr;
  std::map<int, cudaGraphExec_t> stage_graphs;   // graphs of stage subsets, captured on first use
  cudaStream_t own_stream = nullptr;

  int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    err = buf;
    g_last_error = buf;
    return code;
  }
  template <typename T>
  bool dalloc(T** p, size_t count, const char* name = nullptr) {
    void* q = nullptr;
    const size_t nbytes = std::max<size_t>(count * sizeof(T), 256);
    if (cudaMalloc(&q, nbytes) != cudaSuccess) return false;
    cudaMemset(q, 0, nbytes);
    allocs.push_back(q);
    bytes += nbytes;
    *p = reinterpret_cast<T*>(q);
    if (name) named[name] = {q, count * sizeof(T)};
    return true;
  }
};

namespace {

#define CK(call)                                                                                        \
  do {                                                                                                  \
    cudaError_t e_ = (call);                                                                            \
    if (e_ != cudaSuccess) return m->fail(VLA_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(e_)); \
  } while (0)

void add_spec(vla_model* m, const char* key, WKind kind, int which_layers, int K, int N, int lead = 0) {
  WEntry e;
  e.spec = {kind, which_layers >= 0, which_layers, K, N, lead};
  e.L = which_layers == 0 ? m->nvl : (which_layers == 1 ? m->nl : 1);
  e.Kp = round_up(K > 0 ? K : 1, 64);
  e.Np = round_up(N, 128);
  m->W[key] = e;
}

void declare_weights(vla_model* m) {
  // shapes: pi0_infer.py:1245-1287, pi05_infer.py:563-611 of the reference
  add_spec(m, "vision_patch_embedding_w", W_MATRIX, -1, 588, 1152);
  add_spec(m, "vision_patch_embedding_b", W_VECTOR, -1, 0, 1152);
  add_spec(m, "vision_position_embedding", W_VECTOR, -1, 0, 1152, 256);
  add_spec(m, "vision_attn_qkv_w", W_MATRIX, 0, 1152, 3456);
  add_spec(m, "vision_attn_qkv_b", W_VECTOR, 0, 0, 3456);
  add_spec(m, "vision_attn_o_w", W_MATRIX, 0, 1152, 1152);
  add_spec(m, "vision_attn_o_b", W_VECTOR, 0, 0, 1152);
  add_spec(m, "vision_ffn_up_w", W_MATRIX, 0, 1152, 4304);
  add_spec(m, "vision_ffn_up_b", W_VECTOR, 0, 0, 4304);
  add_spec(m, "vision_ffn_down_w", W_MATRIX, 0, 4304, 1152);
  add_spec(m, "vision_ffn_down_b", W_VECTOR, 0, 0, 1152);
  add_spec(m, "vision_pre_attn_norm_w", W_VECTOR, 0, 0, 1152);
  add_spec(m, "vision_pre_attn_norm_b", W_VECTOR, 0, 0, 1152);
  add_spec(m, "vision_pre_ffn_norm_w", W_VECTOR, 0, 0, 1152);
  add_spec(m, "vision_pre_ffn_norm_b", W_VECTOR, 0, 0, 1152);
  add_spec(m, "vision_final_norm_w", W_VECTOR, -1, 0, 1152);
  add_spec(m, "vision_final_norm_b", W_VECTOR, -1, 0, 1152);
  add_spec(m, "encoder_multi_modal_projector_w", W_MATRIX, -1, 1152, 2048);
  add_spec(m, "encoder_multi_modal_projector_b", W_VECTOR, -1, 0, 2048);
  add_spec(m, "encoder_attn_qkv_w", W_MATRIX, 1, 2048, 2560);
  add_spec(m, "encoder_attn_o_w", W_MATRIX, 1, 2048, 2048);
  add_spec(m, "encoder_ffn_gate_w", W_MATRIX, 1, 2048, 16384);
  add_spec(m, "encoder_ffn_up_w", W_MATRIX, 1, 2048, 16384);
  add_spec(m, "encoder_ffn_down_w", W_MATRIX, 1, 16384, 2048);
  add_spec(m, "decoder_attn_qkv_w", W_MATRIX, 1, 1024, 2560);
  add_spec(m, "decoder_attn_o_w", W_MATRIX, 1, 2048, 1024);
  add_spec(m, "decoder_ffn_gate_w", W_MATRIX, 1, 1024, 4096);
  add_spec(m, "decoder_ffn_up_w", W_MATRIX, 1, 1024, 4096);
  add_spec(m, "decoder_ffn_down_w", W_MATRIX, 1, 4096, 1024);
  add_spec(m, "language_embeds", W_PROMPT, -1, 0, 2048);
  if (!m->pi05) {
    add_spec(m, "decoder_state_in_proj_w", W_MATRIX, -1, 32, 1024);
    add_spec(m, "decoder_state_in_proj_b", W_VECTOR, -1, 0, 1024);
    add_spec(m, "decoder_action_fused_in_proj_w", W_MATRIX, -1, 32, 1024);
    add_spec(m, "decoder_action_fused_time_biases", W_VECTOR, -1, 0, 1024, 10);
    add_spec(m, "decoder_action_mlp_w", W_MATRIX, -1, 1024, 1024);
    add_spec(m, "decoder_action_mlp_b", W_VECTOR, -1, 0, 1024);
    add_spec(m, "decoder_action_fused_out_proj_w", W_MATRIX, -1, 1024, 32);
    add_spec(m, "decoder_action_fused_out_proj_b", W_VECTOR, -1, 0, 32);
  } else {
    add_spec(m, "decoder_time_embeds", W_TIME_EMBEDS, -1, 0, 1024, 10);
    add_spec(m, "decoder_time_mlp_in_w", W_MATRIX, -1, 1024, 1024);
    add_spec(m, "decoder_time_mlp_in_b", W_VECTOR, -1, 0, 1024);
    add_spec(m, "decoder_time_mlp_out_w", W_MATRIX, -1, 1024, 1024);
    add_spec(m, "decoder_time_mlp_out_b", W_VECTOR, -1, 0, 1024);
    add_spec(m, "decoder_action_in_proj_w", W_MATRIX, -1, 32, 1024);
    add_spec(m, "decoder_action_in_proj_b", W_VECTOR, -1, 0, 1024);
    add_spec(m, "decoder_pre_attn_norm_mod_w", W_MATRIX, 1, 1024, 3072);
    add_spec(m, "decoder_pre_attn_norm_mod_b", W_VECTOR, 1, 0, 3072);
    add_spec(m, "decoder_pre_ffn_norm_mod_w", W_MATRIX, 1, 1024, 3072);
    add_spec(m, "decoder_pre_ffn_norm_mod_b", W_VECTOR, 1, 0, 3072);
    add_spec(m, "decoder_action_out_proj_w", W_MATRIX, -1, 1024, 32);
    add_spec(m, "decoder_action_out_proj_b", W_VECTOR, -1, 0, 32);
    add_spec(m, "decoder_final_norm_mod_w", W_MATRIX, -1, 1024, 3072);
    add_spec(m, "decoder_final_norm_mod_b", W_VECTOR, -1, 0, 3072);
  }
}

bool alloc_weights(vla_model* m) {
  for (auto& kv : m->W) {
    WEntry& e = kv.second;
    if (e.spec.kind == W_MATRIX) {
      if (!m->dalloc(&e.w, (size_t)e.L * e.Np * e.Kp)) return false;
    } else if (e.spec.kind == W_VECTOR) {
      const int rows = e.spec.layered ? e.L : (e.spec.lead > 0 ? e.spec.lead : 1);
      if (!m->dalloc(&e.v, (size_t)rows * e.Np)) return false;
    }
  }
  return true;
}

bool alloc_buffers(vla_model* m) {
  const size_t B = m->B, Nv = B * m->nv * 256, Np = B * m->P, Ns = B * m->S, Nc = B * m->C;
  bool ok = true;
  ok &= m->dalloc(&m->images, Nv * 588, "observation_images_normalized");
  ok &= m->dalloc(&m->state, B * 32, "observation_state_normalized");
  ok &= m->dalloc(&m->noise, Nc * 32, "diffusion_noise");
  ok &= m->dalloc(&m->noise_f32, Nc * 32);
  ok &= m->dalloc(&m->patches, Nv * 640);
  ok &= m->dalloc(&m->vision_x, Nv * 1152, "vision_x");
  ok &= m->dalloc(&m->vision_xn, Nv * 1152);
  ok &= m->dalloc(&m->vision_qkv, Nv * 3456);
  ok &= m->dalloc(&m->vision_attn, Nv * 1152);
  ok &= m->dalloc(&m->vision_hidden, Nv * 4352);
  ok &= m->dalloc(&m->encoder_x, Np * 2048, "encoder_x");
  ok &= m->dalloc(&m->encoder_xn, Np * 2048);
  ok &= m->dalloc(&m->encoder_q, Np * 2048);
  ok &= m->dalloc(&m->encoder_attn, Np * 2048);
  ok &= m->dalloc(&m->encoder_hidden, Np * 16384);
  ok &= m->dalloc(&m->kcache, (size_t)m->nl * B * m->T * 256, "encoder_K");
  ok &= m->dalloc(&m->vcache, (size_t)m->nl * B * m->T * 256, "encoder_V");
  m->T_pad = round_up(m->T, 8);
  ok &= m->dalloc(&m->vtcache, (size_t)m->nl * B * 256 * m->T_pad);
  ok &= m->dalloc(&m->decoder_x, Ns * 1024, "decoder_x");
  ok &= m->dalloc(&m->state_tok, B * 1024);
  ok &= m->dalloc(&m->decoder_xn, Ns * 1024);
  ok &= m->dalloc(&m->decoder_xb, Ns * 1024);
  ok &= m->dalloc(&m->decoder_ssq, (size_t)32 * Ns);
  ok &= m->dalloc(&m->decoder_q, Ns * 2048, "decoder_q");
  if (B > 1) ok &= m->dalloc(&m->decoder_qkv, Ns * 2560);
  ok &= m->dalloc(&m->decoder_attn, Ns * 2048, "decoder_attn");
  ok &= m->dalloc(&m->decoder_hidden, Ns * 4096, "decoder_hidden");
  ok &= m->dalloc(&m->decoder_act, Nc * 1024, "decoder_act");
  ok &= m->dalloc(&m->decoder_xfin, Nc * 1024);
  ok &= m->dalloc(&m->lang, (size_t)std::max(m->L, 1) * 2048, "language_embeds");
  ok &= m->dalloc(&m->rope_cos, (size_t)(m->T + 1) * 128);
  ok &= m->dalloc(&m->rope_sin, (size_t)(m->T + 1) * 128);
  ok &= m->dalloc(&m->d_valid_len, 4);   // one block: valid length, suffix RoPE start, id count (uploaded together)
  m->d_pos_base = m->d_valid_len + 1;
  m->d_n_ids = m->d_valid_len + 2;
  ok &= m->dalloc(&m->d_status, 1);
  ok &= m->dalloc(&m->d_ids, (size_t)std::max(m->L, 1));
  m->gemm_scratch_cap = (size_t)16 << 20;   // 64 MB: 176 CTAs x the largest partial tile (128 x 256 x 2 fp32)
  ok &= m->dalloc(&m->gemm_scratch, m->gemm_scratch_cap);
  m->attn_scratch_cap = (size_t)6 << 20;    // 24 MB: 176 CTAs x 64 rows x 260 fp32, with headroom
  ok &= m->dalloc(&m->attn_scratch, m->attn_scratch_cap);
  // Persistent action-expert kernel: one observation, suffix rows that fit its shared-memory tile, enough SMs for
  // the feature partition, key splits of at most ATT_MAX_KEYS keys (flags bit 4 keeps the per-operator launches).
  m->use_xp = m->B == 1 && m->S <= xp::MAX_ROWS && m->sm_count >= xp::N_OWNERS && !(m->cfg.flags & 16) && (XP_DEFAULT_ON || (m->cfg.flags & 32));
  if (m->use_xp) {
    xp::Params& xq = m->xp_params;
    memset(&xq, 0, sizeof xq);
    m->xp_G = std::min(m->sm_count, 160);
    xq.att_nrb = (m->S * 8 + xp::ATT_ROWS - 1) / xp::ATT_ROWS;
    xq.att_ks = std::max(1, std::min(m->xp_G / xq.att_nrb, (m->T + 15) / 16));
    xq.att_kps = round_up((m->T + xq.att_ks - 1) / xq.att_ks, 16);
    if (xq.att_kps > xp::ATT_MAX_KEYS) m->use_xp = false;
  }
  if (m->use_xp) {
    const size_t items = (size_t)m->xp_params.att_nrb * m->xp_params.att_ks;
    m->xp_chunks = m->nl * xp::CH_PER_LAYER + 2;
    ok &= m->dalloc(&m->xp_stream, (size_t)m->xp_G * m->xp_chunks * (xp::CHUNK_BYTES / 16));
    ok &= m->dalloc(&m->xp_part, items * xp::ATT_ROWS * 256);
    ok &= m->dalloc(&m->xp_stat, items * xp::ATT_ROWS * 2);
    ok &= m->dalloc(&m->xp_sync, 512);   // barrier counter, abort word, then (at byte 512) the sums of squares [3][64] u64
    ok &= m->dalloc(&m->xp_trace, 4096);
    ok &= m->dalloc(&m->xp_sw_fin, (size_t)10 * 32);
  }
  if (m->pi05) {
    ok &= m->dalloc(&m->style_attn, (size_t)m->nsteps * m->nl * 3072);
    ok &= m->dalloc(&m->style_ffn, (size_t)m->nsteps * m->nl * 3072);
    ok &= m->dalloc(&m->style_fin, (size_t)m->nsteps * 3072);
    ok &= m->dalloc(&m->shift_attn_bf, (size_t)m->nl * m->nsteps * 1024);
    ok &= m->dalloc(&m->shift_ffn_bf, (size_t)m->nl * m->nsteps * 1024);
    ok &= m->dalloc(&m->sw_qkv, (size_t)m->nsteps * m->nl * 2560);
    ok &= m->dalloc(&m->sw_gate, (size_t)m->nsteps * m->nl * 4096);
    ok &= m->dalloc(&m->sw_up, (size_t)m->nsteps * m->nl * 4096);
    ok &= m->dalloc(&m->time_tmp, (size_t)10 * 1024);
    ok &= m->dalloc(&m->time_emb, (size_t)10 * 1024);
  }
  return ok;
}

// ---- plan building -------------------------------------------------------------------------------
struct Plan {
  vla_model* m;
  int stage = 0;
  bool ok = true;
  std::string err;

  void kernel(std::function<cudaError_t(cudaStream_t)> fn) {
    m->ops.push_back({stage, true, std::move(fn)});
    m->n_kernels++;
  }
  GemmEpi epi0() { GemmEpi e; memset(&e, 0, sizeof e); return e; }

  // activations x [tokens, Kx] (pitch ldx) times the layer-l slice of weight `key` (+ `key2` for GeGLU)
  void gemm(const char* key, const char* key2, int layer, const bf16* x, int tokens, int Kx, int ldx, GemmEpi epi,
            int n_feat_override = 0) {
    if (!ok) return;
    WEntry& e = m->W.at(key);
    const bf16* w = e.w + (size_t)layer * e.Np * e.Kp;
    const bf16* w2 = key2 ? m->W.at(key2).w + (size_t)layer * e.Np * e.Kp : nullptr;
    GemmOp op;
    const int n_feat = n_feat_override > 0 ? n_feat_override : e.spec.N;
    if (!build_gemm(&op, w, w2, n_feat, e.Np, e.Kp, x, tokens, Kx, ldx, epi, m->d_status, m->sm_count, 0, 0, &err, 0, 0,
                    (m->cfg.flags & 64) ? 0 : -1)) {
      ok = false;
      err = std::string(key) + ": " + err;
      return;
    }
    if (gemm_scratch_floats(op.bn, op.dual, op.grid, op.p.cg2) > m->gemm_scratch_cap) {
      ok = false;
      err = std::string(key) + ": split-K scratch too small";
      return;
    }
    op.p.scratch = m->gemm_scratch;
    const bool pdl = m->use_pdl;
    kernel([op, pdl](cudaStream_t st) { return launch_gemm(op, st, pdl); });
  }
  const float* vec(const char* key, int layer = 0) {
    WEntry& e = m->W.at(key);
    return e.v + (size_t)layer * e.Np;
  }
  void norm(const float* x, bf16* y, int rows, int D, int mode, const float* w, const float* b, int in_rpo = 0,
            int in_stride = 0, int in_off = 0) {
    const bool pdl = m->use_pdl;
    kernel([=](cudaStream_t st) { return launch_norm(x, D, y, D, rows, D, mode, w, b, in_rpo, in_stride, in_off, st, pdl); });
  }
  // one group per observation: q / o rows g*n_q.., cache rows g*T.., transposed values rows g*256..
  void attention_tc(const bf16* q, const bf16* k, const bf16* vt, bf16* o, int n_q, int n_keys, const int* valid_ptr,
                    int restrict_rows, int groups = 1) {
    if (!ok) return;
    AttnTcOp op;
    const int ks = pick_ksplit_tc(n_q, n_keys, m->sm_count, groups);
    if (attn_tc_scratch_floats(n_q, ks, groups) > m->attn_scratch_cap) { ok = false; err = "attention scratch too small"; return; }
    if (!build_attn_tc(&op, q, k, m->T, vt, m->T_pad, o, 256, n_q, n_keys, m->P, m->P, valid_ptr, restrict_rows, 1.0f / 16.0f,
                       ks, m->attn_scratch, m->d_status, &err, groups, n_q)) {
      ok = false;
      return;
    }
    const bool pdl = m->use_pdl;
    kernel([op, pdl](cudaStream_t st) { return launch_attn_tc(op, st, pdl); });
  }
  void attention(AttnParams p, int head_dim, int groups) {
    const bool pdl = m->use_pdl;
    p.ksplit = pick_ksplit(p.n_q, p.n_keys, groups, m->sm_count);
    p.scratch = m->attn_scratch;
    if (attn_scratch_floats(p, head_dim, groups) > m->attn_scratch_cap) {
      ok = false;
      err = "attention key-split scratch too small";
      return;
    }
    kernel([=](cudaStream_t st) { return launch_attn(p, head_dim, groups, st, pdl); });
  }
};

void plan_vision(Plan& pl) {
  vla_model* m = pl.m;
  pl.stage = 0;
  const bool pdl = m->use_pdl;
  const int Nv = m->B * m->nv * 256;
  {
    const bf16* img = m->images;
    bf16* out = m->patches;
    pl.kernel([=](cudaStream_t st) {
      return launch_ex(patchify_kernel, dim3((Nv * 640 + 255) / 256), dim3(256), 0, st, 1, pdl, img, out, Nv);
    });
  }
  {  // patch embedding + position embedding (pi0_infer.py:348-364)
    GemmEpi e = pl.epi0();
    e.kind = EPI_RESID;
    e.bias = pl.vec("vision_patch_embedding_b");
    e.outf = m->vision_x; e.ld_outf = 1152;
    e.res_in = pl.vec("vision_position_embedding"); e.res_mod = 256; e.ld_res = m->W.at("vision_position_embedding").Np;
    pl.gemm("vision_patch_embedding_w", nullptr, 0, m->patches, Nv, 640, 640, e);
  }
  for (int l = 0; l < m->nvl; ++l) {  // pi0_infer.py:607-646
    pl.norm(m->vision_x, m->vision_xn, Nv, 1152, NORM_LAYER, pl.vec("vision_pre_attn_norm_w", l), pl.vec("vision_pre_attn_norm_b", l));
    GemmEpi e = pl.epi0();
    e.kind = EPI_BF16; e.bias = pl.vec("vision_attn_qkv_b", l); e.out = m->vision_qkv; e.ld_out = 3456;
    pl.gemm("vision_attn_qkv_w", nullptr, l, m->vision_xn, Nv, 1152, 1152, e);
    AttnParams a; memset(&a, 0, sizeof a);
    a.q = m->vision_qkv; a.k = m->vision_qkv + 1152; a.v = m->vision_qkv + 2304; a.o = m->vision_attn;
    a.ldq = a.ldk = a.ldv = 3456; a.ldo = 1152;
    a.q_go = a.k_go = a.v_go = 256LL * 3456; a.q_gi = a.k_gi = a.v_gi = 72; a.o_go = 256LL * 1152; a.o_gi = 72;
    a.g_inner = 16; a.n_q = 256; a.n_keys = 256; a.prefix_alloc = 256; a.valid_prefix = 256; a.restrict_rows = 0;
    a.scale_log2e = 1.4426950408889634f / sqrtf(72.f);
    // One CTA per SM and serial phases make the tcgen05 kernel the faster one for a single observation (latency:
    // vision stage 2.39 -> 2.16 ms at 3 views); with many views in flight the mma.sync kernel, which runs several
    // CTAs per SM, has the higher throughput (64 views: 20.5 against 22.5 ms for the stage), so batches keep it.
    if ((m->cfg.flags & 4) || m->B > 1) {
      pl.attention(a, 72, m->B * m->nv * 16);
    } else {
      VitAttnTcParams vp;
      vp.qkv = m->vision_qkv; vp.o = m->vision_attn; vp.scale_log2e = a.scale_log2e; vp.status = m->d_status; vp.trace = nullptr;
      const int views = m->B * m->nv;
      pl.kernel([=](cudaStream_t st) { return launch_vit_attn_tc(vp, views, st, pdl); });
    }
    e = pl.epi0();
    e.kind = EPI_RESID; e.bias = pl.vec("vision_attn_o_b", l); e.outf = m->vision_x; e.ld_outf = 1152; e.res_in = m->vision_x; e.ld_res = 1152;
    pl.gemm("vision_attn_o_w", nullptr, l, m->vision_attn, Nv, 1152, 1152, e);
    pl.norm(m->vision_x, m->vision_xn, Nv, 1152, NORM_LAYER, pl.vec("vision_pre_ffn_norm_w", l), pl.vec("vision_pre_ffn_norm_b", l));
    e = pl.epi0();
    e.kind = EPI_BF16; e.act = ACT_GELU; e.bias = pl.vec("vision_ffn_up_b", l); e.out = m->vision_hidden; e.ld_out = 4352;
    pl.gemm("vision_ffn_up_w", nullptr, l, m->vision_xn, Nv, 1152, 1152, e, 4352);   // pad columns come out as gelu(0)=0
    e = pl.epi0();
    e.kind = EPI_RESID; e.bias = pl.vec("vision_ffn_down_b", l); e.outf = m->vision_x; e.ld_outf = 1152; e.res_in = m->vision_x; e.ld_res = 1152;
    pl.gemm("vision_ffn_down_w", nullptr, l, m->vision_hidden, Nv, 4352, 4352, e);
  }
  // final LayerNorm + projector into the prefix residual stream (pi0_infer.py:753-775)
  pl.norm(m->vision_x, m->vision_xn, Nv, 1152, NORM_LAYER, pl.vec("vision_final_norm_w"), pl.vec("vision_final_norm_b"));
  GemmEpi e = pl.epi0();
  e.kind = EPI_RESID; e.bias = pl.vec("encoder_multi_modal_projector_b"); e.outf = m->encoder_x; e.ld_outf = 2048;
  e.out_rpo = m->nv * 256; e.out_obs_stride = m->P;
  pl.gemm("encoder_multi_modal_projector_w", nullptr, 0, m->vision_xn, Nv, 1152, 1152, e);
  pl.stage = 1;   // the prompt rows belong to the prefix stage (in multi-GPU latency mode the towers run elsewhere)
  if (m->L > 0 && m->embed_table) {   // prompt given as token ids: embed on the device, inside the graph
    const bf16* table = m->embed_table; const int vocab = m->vocab, L = m->L;
    const int *ids = m->d_ids, *n_ids = m->d_n_ids; bf16* emb = m->lang; int* status = m->d_status;
    pl.kernel([=](cudaStream_t st) {
      return launch_ex(prompt_from_ids_kernel, dim3(L), dim3(256), 0, st, 1, pdl, table, vocab, ids, n_ids, emb,
                       45.254833995939045f, status);
    });
  }
  if (m->L > 0) {  // pi0_infer.py:1344
    const bf16* emb = m->lang; float* x = m->encoder_x;
    const int L = m->L, P = m->P, off = m->nv * 256, B = m->B;
    pl.kernel([=](cudaStream_t st) {
      return launch_ex(prompt_rows_kernel, dim3((unsigned)(((size_t)L * 2048 * B + 255) / 256)), dim3(256), 0, st, 1, pdl, emb, x, L, P, off, B);
    });
  }
}

void plan_prefix(Plan& pl) {
  vla_model* m = pl.m;
  pl.stage = 1;
  const int Np = m->B * m->P;
  for (int l = 0; l < m->nl; ++l) {  // pi0_infer.py:851-884, pi05_infer.py:321-380
    bf16* kc = m->kcache + (size_t)l * m->B * m->T * 256;
    bf16* vc = m->vcache + (size_t)l * m->B * m->T * 256;
    bf16* vt = m->vtcache + (size_t)l * m->B * 256 * m->T_pad;
    pl.norm(m->encoder_x, m->encoder_xn, Np, 2048, NORM_RMS, nullptr, nullptr);
    GemmEpi e = pl.epi0();
    e.kind = EPI_QKV; e.q = m->encoder_q; e.kc = kc; e.vc = vc; e.rope_cos = m->rope_cos; e.rope_sin = m->rope_sin;
    e.vt = vt; e.vt_ld = m->T_pad;
    e.pos_off = 0; e.rows_per_obs = m->P; e.kv_obs_stride = m->T; e.kv_row_off = 0;
    pl.gemm("encoder_attn_qkv_w", nullptr, l, m->encoder_xn, Np, 2048, 2048, e);
    if (l == m->nl - 1) break;   // the last prefix layer only feeds the cache
    AttnParams a; memset(&a, 0, sizeof a);
    a.q = m->encoder_q; a.k = kc; a.v = vc; a.o = m->encoder_attn;
    a.ldq = a.ldk = a.ldv = a.ldo = 256;
    a.q_go = a.o_go = (long long)m->P * 2048; a.k_go = a.v_go = (long long)m->T * 256;
    a.g_inner = 1; a.n_q = m->P * 8; a.n_keys = m->P; a.prefix_alloc = m->P; a.valid_prefix = m->P;
    a.valid_prefix_ptr = m->pi05 ? m->d_valid_len : nullptr;
    a.scale_log2e = 1.4426950408889634f / 16.f;
    if (m->B == 1 || !(m->cfg.flags & 8)) pl.attention_tc(m->encoder_q, kc, vt, m->encoder_attn, m->P * 8, m->P, m->pi05 ? m->d_valid_len : nullptr, 0, m->B);
    else pl.attention(a, 256, m->B);
    e = pl.epi0();
    e.kind = EPI_RESID; e.outf = m->encoder_x; e.ld_outf = 2048; e.res_in = m->encoder_x; e.ld_res = 2048;
    pl.gemm("encoder_attn_o_w", nullptr, l, m->encoder_attn, Np, 2048, 2048, e);
    pl.norm(m->encoder_x, m->encoder_xn, Np, 2048, NORM_RMS, nullptr, nullptr);
    e = pl.epi0();
    e.kind = EPI_BF16; e.act = ACT_GEGLU; e.out = m->encoder_hidden; e.ld_out = 16384;
    pl.gemm("encoder_ffn_gate_w", "encoder_ffn_up_w", l, m->encoder_xn, Np, 2048, 2048, e);
    e = pl.epi0();
    e.kind = EPI_RESID; e.outf = m->encoder_x; e.ld_outf = 2048; e.res_in = m->encoder_x; e.ld_res = 2048;
    pl.gemm("encoder_ffn_down_w", nullptr, l, m->encoder_hidden, Np, 16384, 16384, e);
  }
}

// ---- persistent action-expert kernel ---------------------------------------------------------------
// Repack the expert's weights (already K-major in W[...]) into the per-CTA streams the kernel reads.
int xp_pack(vla_model* m) {
  const int G = m->xp_G;
  bf16* stream = reinterpret_cast<bf16*>(m->xp_stream);
  const size_t chunk_elems = xp::CHUNK_BYTES / 2;
  auto layer_w = [&](const char* key, int l) {
    WEntry& e = m->W.at(key);
    return e.w + (size_t)l * e.Np * e.Kp;
  };
  for (int l = 0; l < m->nl; ++l)
    xp::pack_layer_kernel<<<dim3(xp::CH_PER_LAYER, G), 256>>>(layer_w("decoder_attn_qkv_w", l), layer_w("decoder_attn_o_w", l),
                                                              layer_w("decoder_ffn_gate_w", l), layer_w("decoder_ffn_up_w", l),
                                                              layer_w("decoder_ffn_down_w", l), l, m->xp_chunks, stream);
  const int misc = m->nl * xp::CH_PER_LAYER;
  if (!m->pi05)
    for (int c = 0; c < xp::N_OWNERS; ++c)
      xp::pack_chunk_kernel<<<32, 256>>>(m->W.at("decoder_action_mlp_w").w, 1024, 1024, 1024, 8 * c, 0,
                                         stream + ((size_t)c * m->xp_chunks + misc) * chunk_elems);
  const WEntry& wo = m->W.at(m->pi05 ? "decoder_action_out_proj_w" : "decoder_action_fused_out_proj_w");
  for (int c = 0; c < 4; ++c)
    xp::pack_chunk_kernel<<<32, 256>>>(wo.w, wo.Kp, 32, 1024, 8 * c, 0, stream + ((size_t)c * m->xp_chunks + misc + 1) * chunk_elems);
  CK(cudaGetLastError());
  CK(cudaDeviceSynchronize());
  return VLA_OK;
}

cudaError_t launch_expert_persistent(vla_model* m, cudaStream_t st, unsigned long long* trace) {
  auto kern = xp::expert_persistent_kernel;
  if (cudaError_t e = ensure_smem_attr(reinterpret_cast<const void*>(kern), xp::SMEM_BYTES); e != cudaSuccess) return e;
  // barrier counter and abort word start from zero at every launch
  if (cudaError_t e = cudaMemsetAsync(m->xp_sync, 0, 512 * sizeof(unsigned int), st); e != cudaSuccess) return e;
  xp::Params p = m->xp_params;
  p.trace = trace;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof cfg);
  cfg.gridDim = dim3(m->xp_G);
  cfg.blockDim = dim3(xp::THREADS);
  cfg.dynamicSmemBytes = xp::SMEM_BYTES;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;   // all CTAs co-resident: they wait for one another at grid barriers
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, p);
}

void plan_decoder_persistent(Plan& pl) {
  vla_model* m = pl.m;
  pl.stage = 2;
  const bool pi05 = m->pi05;
  xp::Params& p = m->xp_params;   // attention split already chosen in alloc_buffers
  p.pi05 = pi05; p.S = m->S; p.C = m->C; p.P = m->P; p.T = m->T; p.nl = m->nl; p.nsteps = m->nsteps; p.G = m->xp_G;
  p.wstream = m->xp_stream; p.chunks_per_cta = m->xp_chunks; p.misc_base = m->nl * xp::CH_PER_LAYER;
  if (pi05) {
    p.w_in = m->W.at("decoder_action_in_proj_w").w;
    p.b_in = pl.vec("decoder_action_in_proj_b"); p.ld_b_in = 0;
    p.b_out = pl.vec("decoder_action_out_proj_b");
    p.sw_fin = m->xp_sw_fin;
    p.style_attn = m->style_attn; p.style_ffn = m->style_ffn; p.style_fin = m->style_fin;
    p.sw_qkv = m->sw_qkv; p.sw_gate = m->sw_gate; p.sw_up = m->sw_up;
    p.valid_len_ptr = m->d_valid_len; p.pos_base_ptr = m->d_pos_base;
  } else {
    p.w_in = m->W.at("decoder_action_fused_in_proj_w").w;
    p.b_in = pl.vec("decoder_action_fused_time_biases"); p.ld_b_in = m->W.at("decoder_action_fused_time_biases").Np;
    p.b_mlp = pl.vec("decoder_action_mlp_b");
    p.w_state = m->W.at("decoder_state_in_proj_w").w; p.b_state = pl.vec("decoder_state_in_proj_b"); p.state = m->state;
    p.b_out = pl.vec("decoder_action_fused_out_proj_b");
  }
  p.noise = m->noise; p.noise_f32 = m->noise_f32; p.act = m->decoder_act; p.x_out = m->decoder_x; p.xb = m->decoder_xb;
  p.ssq = reinterpret_cast<unsigned long long*>(m->xp_sync + 128); p.q = m->decoder_q; p.kcache = m->kcache; p.vcache = m->vcache; p.attn = m->decoder_attn;
  p.hidden = m->decoder_hidden; p.att_part = m->xp_part; p.att_stat = m->xp_stat;
  p.rope_cos = m->rope_cos; p.rope_sin = m->rope_sin;
  p.bar_ctr = m->xp_sync; p.status = m->d_status; p.trace = nullptr;
  // activation operands come in by TMA: four 64-wide K blocks of MAX_ROWS rows per copy, 128-byte swizzle
  const bool maps_ok =
      make_tmap3(&p.tm_xb, m->decoder_xb, 1024, m->S, 1024, xp::MAX_ROWS, 4, &pl.err) &&
      make_tmap3(&p.tm_act, m->decoder_act, 1024, m->C, 1024, xp::MAX_ROWS, 4, &pl.err) &&
      make_tmap3(&p.tm_attn, m->decoder_attn, 2048, m->S, 2048, xp::MAX_ROWS, 4, &pl.err) &&
      make_tmap3(&p.tm_hidden, m->decoder_hidden, 4096, m->S, 4096, xp::MAX_ROWS, 4, &pl.err) &&
      make_tmap3(&p.tm_q, m->decoder_q, 256, m->S * 8, 256, xp::ATT_ROWS, 4, &pl.err) &&
      make_tmap3(&p.tm_k, m->kcache, 256, (long long)m->nl * m->T, 256, p.att_kps, 4, &pl.err) &&
      make_tmap3(&p.tm_v, m->vcache, 256, (long long)m->nl * m->T, 256, p.att_kps, 4, &pl.err);
  if (!maps_ok) { pl.ok = false; return; }
  pl.kernel([m](cudaStream_t st) { return launch_expert_persistent(m, st, nullptr); });
}

void plan_decoder(Plan& pl) {
  vla_model* m = pl.m;
  if (m->use_xp) { plan_decoder_persistent(pl); return; }
  pl.stage = 2;
  const bool pdl = m->use_pdl, pi05 = m->pi05;
  const int Ns = m->B * m->S, Nc = m->B * m->C, B = m->B, S = m->S, C = m->C;
  {
    const bf16* nz = m->noise; float* nf = m->noise_f32;
    pl.kernel([=](cudaStream_t st) {
      return launch_ex(noise_init_kernel, dim3((Nc * 32 + 255) / 256), dim3(256), 0, st, 1, pdl, nz, nf, Nc * 32);
    });
  }
  if (!pi05) {  // state token, once per forward (pi0_infer.py:1166-1171)
    GemmEpi e = pl.epi0();
    e.kind = EPI_RESID; e.bias = pl.vec("decoder_state_in_proj_b"); e.outf = m->state_tok; e.ld_outf = 1024;
    pl.gemm("decoder_state_in_proj_w", nullptr, 0, m->state, B, 32, 32, e);
  }
  for (int step = 0; step < m->nsteps; ++step) {
    if (!pi05) {  // pi0_infer.py:1173-1185
      const float* src = m->state_tok; float* dst = m->decoder_x;
      pl.kernel([=](cudaStream_t st) {
        return launch_ex(copy_rows_kernel, dim3((1024 * B + 255) / 256), dim3(256), 0, st, 1, pdl, src, dst, 1024, S, 0, B);
      });
      GemmEpi e = pl.epi0();
      e.kind = EPI_BF16; e.act = ACT_SILU; e.bias = pl.vec("decoder_action_fused_time_biases", step % 10);
      e.out = m->decoder_act; e.ld_out = 1024;
      pl.gemm("decoder_action_fused_in_proj_w", nullptr, 0, m->noise, Nc, 32, 32, e);
      e = pl.epi0();
      e.kind = EPI_RESID; e.bias = pl.vec("decoder_action_mlp_b"); e.outf = m->decoder_x + 1024; e.ld_outf = 1024;
      e.out_rpo = C; e.out_obs_stride = S;
      pl.gemm("decoder_action_mlp_w", nullptr, 0, m->decoder_act, Nc, 1024, 1024, e);
    } else {      // pi05_infer.py:420-425
      GemmEpi e = pl.epi0();
      e.kind = EPI_RESID; e.bias = pl.vec("decoder_action_in_proj_b"); e.outf = m->decoder_x; e.ld_outf = 1024;
      pl.gemm("decoder_action_in_proj_w", nullptr, 0, m->noise, Nc, 32, 32, e);
    }
    for (int l = 0; l < m->nl; ++l) {  // pi0_infer.py:1186-1223, pi05_infer.py:427-509
      bf16* kc = m->kcache + (size_t)l * B * m->T * 256;
      bf16* vc = m->vcache + (size_t)l * B * m->T * 256;
      bf16* vt = m->vtcache + (size_t)l * B * 256 * m->T_pad;
      const float* st_attn = pi05 ? m->style_attn + ((size_t)step * m->nl + l) * 3072 : nullptr;
      const float* st_ffn = pi05 ? m->style_ffn + ((size_t)step * m->nl + l) * 3072 : nullptr;
      // The RMS norms are folded into the GEMMs (f * (x @ W)); only the first layer of a step normalises
      // explicitly, because its input comes from the action MLP.  Pi05 (adaRMS): the producer's bf16 mirror holds
      // x * (1 + scale) of the norm that consumes it and the consumer adds the precomputed shift @ W as a bias.
      // Batched forwards do not fold: the producer side of the fold (bf16 mirror + per-token sums of squares) keeps the
      // residual GEMMs on the per-column epilogue, which at 1632 tokens costs more (39 us per launch) than two norm
      // launches and the tile-store epilogue (in-place fp32 reduce-add through TMA) together.
      const bool fold = B == 1;
      const bool explicit_norm = !fold || l == 0;
      const size_t sl = (size_t)step * m->nl + l;
      if (explicit_norm) pl.norm(m->decoder_x, m->decoder_xn, Ns, 1024, pi05 ? NORM_ADARMS : NORM_RMS, st_attn, nullptr);
      GemmEpi e = pl.epi0();
      e.kind = EPI_QKV; e.q = m->decoder_q; e.kc = kc; e.vc = vc; e.rope_cos = m->rope_cos; e.rope_sin = m->rope_sin;
      e.pos_off = pi05 ? 0 : m->P; e.pos_base = pi05 ? m->d_pos_base : nullptr;
      e.rows_per_obs = S; e.kv_obs_stride = m->T; e.kv_row_off = m->P;
      e.vt = vt; e.vt_ld = m->T_pad;
      if (!explicit_norm) {
        e.ssq_in = m->decoder_ssq; e.ssq_ld = Ns; e.ssq_slots = 32; e.ssq_inv_d = 1.0f / 1024.0f;
        if (pi05) e.bias = m->sw_qkv + sl * 2560;
      }
      if (B > 1) {
        // batched: plain GEMM into a bf16 buffer (tile stores), then rotary embedding and cache append as one
        // coalesced pass; the fused epilogue would run per column here (38 us per launch against 12 + 5)
        GemmEpi g = pl.epi0();
        g.kind = EPI_BF16; g.out = m->decoder_qkv; g.ld_out = 2560;
        pl.gemm("decoder_attn_qkv_w", nullptr, l, m->decoder_xn, Ns, 1024, 1024, g);
        const bf16* src = m->decoder_qkv; bf16* qd = m->decoder_q;
        const float *rc = m->rope_cos, *rs = m->rope_sin;
        const int po = e.pos_off, T = m->T, P = m->P, vt_ld = m->T_pad;
        const int* pbase = e.pos_base;
        pl.kernel([=](cudaStream_t st) {
          return launch_ex(qkv_rope_split_kernel, dim3((Ns + 31) / 32, 5), dim3(256), 0, st, 1, pdl, src, Ns, qd, kc, vc, vt, vt_ld, rc, rs,
                           po, pbase, S, T, P);
        });
      } else {
        pl.gemm("decoder_attn_qkv_w", nullptr, l, explicit_norm ? m->decoder_xn : m->decoder_xb, Ns, 1024, 1024, e);
      }
      AttnParams a; memset(&a, 0, sizeof a);
      a.q = m->decoder_q; a.k = kc; a.v = vc; a.o = m->decoder_attn;
      a.ldq = a.ldk = a.ldv = a.ldo = 256;
      a.q_go = a.o_go = (long long)S * 2048; a.k_go = a.v_go = (long long)m->T * 256;
      a.g_inner = 1; a.n_q = S * 8; a.n_keys = m->T; a.prefix_alloc = m->P; a.valid_prefix = m->P;
      a.valid_prefix_ptr = pi05 ? m->d_valid_len : nullptr;
      a.restrict_rows = pi05 ? 0 : 8;
      a.scale_log2e = 1.4426950408889634f / 16.f;
      if (B == 1 || !(m->cfg.flags & 8)) pl.attention_tc(m->decoder_q, kc, vt, m->decoder_attn, S * 8, m->T, pi05 ? m->d_valid_len : nullptr, pi05 ? 0 : 8, B);
      else pl.attention(a, 256, B);
      e = pl.epi0();
      e.kind = EPI_RESID; e.outf = m->decoder_x; e.ld_outf = 1024; e.res_in = m->decoder_x; e.ld_res = 1024;
      e.gate = pi05 ? st_attn + 2048 : nullptr;
      if (fold) { e.mirror = m->decoder_xb; e.ld_mirror = 1024; e.ssq_out = m->decoder_ssq; e.ssq_ld = Ns; }
      if (pi05 && fold) e.mirror_scale = st_ffn;   // scale third of the pre-MLP norm's style row
      pl.gemm("decoder_attn_o_w", nullptr, l, m->decoder_attn, Ns, 2048, 2048, e);
      if (!fold) pl.norm(m->decoder_x, m->decoder_xn, Ns, 1024, pi05 ? NORM_ADARMS : NORM_RMS, st_ffn, nullptr);
      e = pl.epi0();
      e.kind = EPI_BF16; e.act = ACT_GEGLU; e.out = m->decoder_hidden; e.ld_out = 4096;
      if (fold) { e.ssq_in = m->decoder_ssq; e.ssq_ld = Ns; e.ssq_slots = 32; e.ssq_inv_d = 1.0f / 1024.0f; }
      if (pi05 && fold) { e.bias = m->sw_gate + sl * 4096; e.bias2 = m->sw_up + sl * 4096; }
      pl.gemm("decoder_ffn_gate_w", "decoder_ffn_up_w", l, fold ? m->decoder_xb : m->decoder_xn, Ns, 1024, 1024, e);
      e = pl.epi0();
      e.kind = EPI_RESID; e.outf = m->decoder_x; e.ld_outf = 1024; e.res_in = m->decoder_x; e.ld_res = 1024;
      e.gate = pi05 ? st_ffn + 2048 : nullptr;
      if (fold) { e.mirror = m->decoder_xb; e.ld_mirror = 1024; e.ssq_out = m->decoder_ssq; e.ssq_ld = Ns; }
      if (pi05 && fold && l + 1 < m->nl) e.mirror_scale = st_attn + 3072;   // pre-attention norm of the next layer, same step
      pl.gemm("decoder_ffn_down_w", nullptr, l, m->decoder_hidden, Ns, 4096, 4096, e);
    }
    // Euler update: noise += norm(x_action) @ W_out + b_out   (pi0_infer.py:1224-1230, pi05_infer.py:511-523)
    if (!pi05) pl.norm(m->decoder_x, m->decoder_xfin, Nc, 1024, NORM_RMS, nullptr, nullptr, C, S, 1);
    else pl.norm(m->decoder_x, m->decoder_xfin, Nc, 1024, NORM_ADARMS, m->style_fin + (size_t)step * 3072, nullptr);
    GemmEpi e = pl.epi0();
    e.kind = EPI_RESID; e.outf = m->noise_f32; e.ld_outf = 32; e.res_in = m->noise_f32; e.ld_res = 32;
    e.mirror = m->noise; e.ld_mirror = 32;
    e.bias = pl.vec(pi05 ? "decoder_action_out_proj_b" : "decoder_action_fused_out_proj_b");
    pl.gemm(pi05 ? "decoder_action_out_proj_w" : "decoder_action_fused_out_proj_w", nullptr, 0, m->decoder_xfin, Nc, 1024, 1024, e);
  }
}

int run_ops(vla_model* m, cudaStream_t st, int stage_filter = -1) {
  for (auto& op : m->ops) {
    if (stage_filter >= 0 && op.stage != stage_filter) continue;
    cudaError_t e = op.fn(st);
    if (e != cudaSuccess) return m->fail(VLA_ERR_CUDA, "launch failed in stage %d: %s", op.stage, cudaGetErrorString(e));
  }
  return VLA_OK;
}

// Pi05 constructor-time work: scaled out-projection, time MLP, adaRMS style rows (pi05_infer.py:669-722)
int pi05_precompute(vla_model* m, cudaStream_t st) {
  Plan pl{m};
  std::vector<vla_model::Op> saved;
  saved.swap(m->ops);
  const int saved_n = m->n_kernels;
  const int ns = m->nsteps;
  const bf16* te = reinterpret_cast<const bf16*>(m->named["decoder_time_embeds"].first);
  GemmEpi e = pl.epi0();
  e.kind = EPI_BF16; e.act = ACT_SILU; e.bias = pl.vec("decoder_time_mlp_in_b"); e.out = m->time_tmp; e.ld_out = 1024;
  pl.gemm("decoder_time_mlp_in_w", nullptr, 0, te, ns, 1024, 1024, e);
  e.bias = pl.vec("decoder_time_mlp_out_b"); e.out = m->time_emb;
  pl.gemm("decoder_time_mlp_out_w", nullptr, 0, m->time_tmp, ns, 1024, 1024, e);
  for (int l = 0; l < m->nl; ++l) {
    GemmEpi s = pl.epi0();
    s.kind = EPI_RESID; s.bias = pl.vec("decoder_pre_attn_norm_mod_b", l); s.outf = m->style_attn + (size_t)l * 3072; s.ld_outf = m->nl * 3072;
    pl.gemm("decoder_pre_attn_norm_mod_w", nullptr, l, m->time_emb, ns, 1024, 1024, s);
    s.bias = pl.vec("decoder_pre_ffn_norm_mod_b", l); s.outf = m->style_ffn + (size_t)l * 3072;
    pl.gemm("decoder_pre_ffn_norm_mod_w", nullptr, l, m->time_emb, ns, 1024, 1024, s);
  }
  GemmEpi s = pl.epi0();
  s.kind = EPI_RESID; s.bias = pl.vec("decoder_final_norm_mod_b"); s.outf = m->style_fin; s.ld_outf = 3072;
  pl.gemm("decoder_final_norm_mod_w", nullptr, 0, m->time_emb, ns, 1024, 1024, s);
  // The adaRMS norms of the expert are folded into the GEMMs that consume them:
  //   (rms(x) * (1 + scale) + shift) @ W = f * ((x * (1 + scale)) @ W) + shift @ W,  f = rsqrt(mean(x^2) + eps),
  // so shift @ W is computed here once per (step, layer) and enters the GEMM epilogues as a bias.
  {
    const int nl = m->nl;
    const unsigned blocks = (unsigned)(((size_t)nl * ns * 1024 + 255) / 256);
    const float *sa = m->style_attn, *sf = m->style_ffn;
    bf16 *oa = m->shift_attn_bf, *of = m->shift_ffn_bf;
    pl.kernel([=](cudaStream_t st2) { style_shift_rows_kernel<<<blocks, 256, 0, st2>>>(sa, nl, ns, oa); return cudaGetLastError(); });
    pl.kernel([=](cudaStream_t st2) { style_shift_rows_kernel<<<blocks, 256, 0, st2>>>(sf, nl, ns, of); return cudaGetLastError(); });
    for (int l = 0; l < nl; ++l) {
      GemmEpi b = pl.epi0();
      b.kind = EPI_RESID; b.outf = m->sw_qkv + (size_t)l * 2560; b.ld_outf = nl * 2560;
      pl.gemm("decoder_attn_qkv_w", nullptr, l, m->shift_attn_bf + (size_t)l * ns * 1024, ns, 1024, 1024, b);
      b.outf = m->sw_gate + (size_t)l * 4096; b.ld_outf = nl * 4096;
      pl.gemm("decoder_ffn_gate_w", nullptr, l, m->shift_ffn_bf + (size_t)l * ns * 1024, ns, 1024, 1024, b);
      b.outf = m->sw_up + (size_t)l * 4096;
      pl.gemm("decoder_ffn_up_w", nullptr, l, m->shift_ffn_bf + (size_t)l * ns * 1024, ns, 1024, 1024, b);
    }
  }
  if (m->use_xp) {   // shift @ W of the final adaRMS norm, folded into the out-projection of the persistent kernel
    const float* sf = m->style_fin; const bf16* wo = m->W.at("decoder_action_out_proj_w").w; const int kp = m->W.at("decoder_action_out_proj_w").Kp;
    float* out = m->xp_sw_fin;
    pl.kernel([=](cudaStream_t st2) { xp::sw_fin_kernel<<<ns, 1024, 0, st2>>>(sf, wo, kp, ns, out); return cudaGetLastError(); });
  }
  int rc = VLA_OK;
  if (!pl.ok) rc = m->fail(VLA_ERR_CUDA, "pi05 precompute plan: %s", pl.err.c_str());
  else rc = run_ops(m, st);
  m->ops.swap(saved);
  m->n_kernels = saved_n;
  if (rc) return rc;
  CK(cudaStreamSynchronize(st));
  return VLA_OK;
}

int check_status(vla_model* m) {
  int w = 0;
  CK(cudaMemcpy(&w, m->d_status, sizeof w, cudaMemcpyDeviceToHost));
  if (w) return m->fail(VLA_ERR_DEVICE, "device status word 0x%x (bounded wait timed out or bad shape)", w);
  return VLA_OK;
}

}  // namespace

// ===================================================================================================
extern "C" {

const char* vla_last_error(vla_handle h) { return h ? h->err.c_str() : g_last_error.c_str(); }

int vla_create(const vla_config* cfg, vla_handle* out) {
  if (!cfg || !out) { g_last_error = "null argument"; return VLA_ERR_STATE; }
  *out = nullptr;
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
    cudaGetLastError();
    g_last_error = "no CUDA device: libvla_b200 has no CPU path";
    return VLA_ERR_CUDA;
  }
  vla_model* m = new vla_model();
  m->cfg = *cfg;
  auto bail = [&](int code) { g_last_error = m->err; vla_destroy(m); return code; };
  if (cfg->device < 0 || cfg->device >= ndev) return bail(m->fail(VLA_ERR_SHAPE, "device %d out of range", cfg->device));
  if (cudaSetDevice(cfg->device) != cudaSuccess) return bail(m->fail(VLA_ERR_CUDA, "cudaSetDevice failed"));
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, cfg->device) != cudaSuccess) return bail(m->fail(VLA_ERR_CUDA, "cudaGetDeviceProperties failed"));
  if (prop.major != 10) return bail(m->fail(VLA_ERR_CUDA, "device is sm_%d%d; this library is built for sm_100a only", prop.major, prop.minor));
  m->sm_count = prop.multiProcessorCount;
  m->pi05 = cfg->model == VLA_PI05;
  m->nv = cfg->num_views; m->C = cfg->chunk_size; m->L = cfg->prompt_len; m->B = cfg->batch > 0 ? cfg->batch : 1;
  m->nvl = cfg->n_vit_layers > 0 ? cfg->n_vit_layers : 27;
  m->nl = cfg->n_layers > 0 ? cfg->n_layers : 18;
  m->nsteps = cfg->n_steps > 0 ? cfg->n_steps : 10;
  if (cfg->model != VLA_PI0 && cfg->model != VLA_PI05) return bail(m->fail(VLA_ERR_SHAPE, "unknown model kind %d", cfg->model));
  if (m->nv < 1 || m->nv > 8 || m->C < 1 || m->L < 0) return bail(m->fail(VLA_ERR_SHAPE, "bad num_views/chunk_size/prompt_len"));
  if (m->nvl > 27 || m->nl > 18 || m->nsteps > 10) return bail(m->fail(VLA_ERR_SHAPE, "layer/step counts exceed the model's"));
  m->P = m->nv * 256 + m->L;
  m->S = m->C + (m->pi05 ? 0 : 1);
  m->T = m->P + m->S;
  // the reference's softmax kernels hold one row of <= 1024 keys (pi0_infer.py:1073,1106; pi05_infer.py:295,397)
  if (m->T > 1024) return bail(m->fail(VLA_ERR_LIMIT, "prefix + suffix = %d keys exceeds the 1024-key limit of the path", m->T));
  m->valid_len = m->P;
  m->use_pdl = !(cfg->flags & 1);
  m->use_graph = !(cfg->flags & 2);
  declare_weights(m);
  if (!alloc_weights(m) || !alloc_buffers(m)) return bail(m->fail(VLA_ERR_CUDA, "device allocation failed: %s", cudaGetErrorString(cudaGetLastError())));
  if (cudaStreamCreateWithFlags(&m->own_stream, cudaStreamNonBlocking) != cudaSuccess) return bail(m->fail(VLA_ERR_CUDA, "stream creation failed"));
  *out = m;
  return VLA_OK;
}

int vla_load_weight(vla_handle m, const char* key, const void* data, const int64_t* shape, int ndim, int dtype) {
  if (!m) return VLA_ERR_STATE;
  if (!key || !shape) return m->fail(VLA_ERR_STATE, "null key or shape");
  cudaSetDevice(m->cfg.device);
  if (!strcmp(key, "embedding_weight")) {
    // token embedding table of the prompt (pi05_infer.py:726-743): kept as bf16 [vocab, 2048], used by
    // vla_set_prompt_ids; must be loaded before vla_finalize so that the gather is part of the graph
    if (m->finalized) return m->fail(VLA_ERR_STATE, "'embedding_weight' must be loaded before vla_finalize");
    if (ndim != 2 || shape[1] != 2048 || shape[0] < 1 || shape[0] > (1 << 24))
      return m->fail(VLA_ERR_SHAPE, "'embedding_weight' must be (vocab, 2048)");
    if (dtype != VLA_BF16 && dtype != VLA_F32) return m->fail(VLA_ERR_SHAPE, "'%s': dtype must be bf16 or f32", key);
    if (!data) return m->fail(VLA_ERR_STATE, "'%s': null data pointer", key);
    const size_t count = (size_t)shape[0] * 2048;
    if (m->embed_table) return m->fail(VLA_ERR_STATE, "'embedding_weight' is already loaded");
    if (!m->dalloc(&m->embed_table, count)) return m->fail(VLA_ERR_CUDA, "allocation of the embedding table failed");
    if (dtype == VLA_BF16) {
      CK(cudaMemcpy(m->embed_table, data, count * 2, cudaMemcpyDefault));
    } else {
      float* raw = nullptr;
      CK(cudaMalloc(&raw, count * 4));
      cudaError_t ce = cudaMemcpy(raw, data, count * 4, cudaMemcpyDefault);
      if (ce == cudaSuccess) {
        f32_to_bf16_kernel<<<(unsigned)((count + 255) / 256), 256>>>(raw, m->embed_table, count);
        ce = cudaDeviceSynchronize();
      }
      cudaFree(raw);
      if (ce != cudaSuccess) return m->fail(VLA_ERR_CUDA, "embedding table upload: %s", cudaGetErrorString(ce));
    }
    m->vocab = (int)shape[0];
    return VLA_OK;
  }
  auto it = m->W.find(key);
  if (it == m->W.end()) return m->fail(VLA_ERR_KEY, "unknown checkpoint key '%s'", key);
  WEntry& e = it->second;
  size_t count = 1;
  for (int i = 0; i < ndim; ++i) count *= (size_t)shape[i];
  // expected element count
  size_t expect;
  if (e.spec.kind == W_MATRIX) expect = (size_t)e.L * e.spec.K * e.spec.N;
  else if (e.spec.kind == W_VECTOR) expect = (size_t)(e.spec.layered ? e.L : (e.spec.lead > 0 ? e.spec.lead : 1)) * e.spec.N;
  else if (e.spec.kind == W_TIME_EMBEDS) expect = (size_t)10 * 1024;
  else expect = (size_t)m->L * 2048;
  if (e.spec.kind == W_PROMPT) {
    if (ndim != 2 || shape[1] != 2048 || shape[0] > m->L)
      return m->fail(VLA_ERR_SHAPE, "language_embeds must be (<=%d, 2048)", m->L);
    expect = count;
  }
  if (count != expect) return m->fail(VLA_ERR_SHAPE, "'%s': got %zu elements, expected %zu", key, count, expect);
  if (dtype != VLA_BF16 && dtype != VLA_F32) return m->fail(VLA_ERR_SHAPE, "'%s': dtype must be bf16 or f32", key);
  if (count == 0) { e.loaded = true; return VLA_OK; }
  if (!data) return m->fail(VLA_ERR_STATE, "'%s': null data pointer", key);

  // stage the raw tensor on the device as bf16
  const size_t esz = dtype == VLA_BF16 ? 2 : 4;
  void* raw = nullptr;
  CK(cudaMalloc(&raw, count * esz));
  cudaError_t ce = cudaMemcpy(raw, data, count * esz, cudaMemcpyDefault);
  bf16* stage = reinterpret_cast<bf16*>(raw);
  void* conv = nullptr;
  if (ce == cudaSuccess && dtype == VLA_F32) {
    ce = cudaMalloc(&conv, count * 2);
    if (ce == cudaSuccess) {
      f32_to_bf16_kernel<<<(unsigned)((count + 255) / 256), 256>>>(reinterpret_cast<float*>(raw), reinterpret_cast<bf16*>(conv), count);
      stage = reinterpret_cast<bf16*>(conv);
      ce = cudaGetLastError();
    }
  }
  if (ce == cudaSuccess) {
    if (e.spec.kind == W_MATRIX) {
      // Pi05 scales the out-projection by -1/steps in place, in bf16, at construction (pi05_infer.py:670-671)
      if (m->pi05 && !strncmp(key, "decoder_action_out_proj", 23))
        scale_bf16_kernel<<<(unsigned)((count + 255) / 256), 256>>>(stage, count, -1.0f / 10.0f);
      for (int l = 0; l < e.L; ++l) {
        dim3 grid((e.Np + 31) / 32, (e.Kp + 31) / 32), block(32, 8);
        repack_kn_to_nk<<<grid, block>>>(stage + (size_t)l * e.spec.K * e.spec.N, e.spec.K, e.spec.N,
                                         e.w + (size_t)l * e.Np * e.Kp, e.Kp, e.Np);
      }
    } else if (e.spec.kind == W_VECTOR) {
      const int rows = e.spec.layered ? e.L : (e.spec.lead > 0 ? e.spec.lead : 1);
      float scale = 1.0f;
      if (m->pi05 && !strncmp(key, "decoder_action_out_proj", 23)) {
        scale_bf16_kernel<<<(unsigned)((count + 255) / 256), 256>>>(stage, count, -1.0f / 10.0f);
      }
      for (int r = 0; r < rows; ++r)
        bf16_to_f32_kernel<<<(e.spec.N + 255) / 256, 256>>>(stage + (size_t)r * e.spec.N, e.v + (size_t)r * e.Np, e.spec.N, scale);
    } else if (e.spec.kind == W_TIME_EMBEDS) {
      bf16* dst = nullptr;
      auto f = m->named.find(key);
      if (f == m->named.end()) { if (m->dalloc(&dst, count, key)) {} } else dst = reinterpret_cast<bf16*>(f->second.first);
      if (dst) ce = cudaMemcpy(dst, stage, count * 2, cudaMemcpyDeviceToDevice); else ce = cudaErrorMemoryAllocation;
    } else {  // prompt
      ce = cudaMemset(m->lang, 0, (size_t)std::max(m->L, 1) * 2048 * 2);
      if (ce == cudaSuccess) ce = cudaMemcpy(m->lang, stage, count * 2, cudaMemcpyDeviceToDevice);
      m->valid_len = m->nv * 256 + (int)shape[0];
    }
    if (ce == cudaSuccess) ce = cudaGetLastError();
    if (ce == cudaSuccess) ce = cudaDeviceSynchronize();
  }
  cudaFree(raw);
  if (conv) cudaFree(conv);
  if (ce != cudaSuccess) return m->fail(VLA_ERR_CUDA, "'%s': upload/repack failed: %s", key, cudaGetErrorString(ce));
  e.loaded = true;
  return VLA_OK;
}

// Every update below is enqueued on `st`, so it is ordered after a forward already running on that stream and
// before the next one (the reference's fill_/copy_ are stream-ordered the same way, pi05_infer.py:819-822).  The
// three scalars travel as one 12-byte copy from a pinned staging slot of the handle; slots rotate so that a slot is
// not rewritten while an earlier copy may still be reading it.
static int upload_scalars(vla_model* m, cudaStream_t st) {
  // Pi05: valid prefix length and suffix RoPE start (pi05_infer.py:787-790, 821); Pi0: fixed
  if (!m->h_scalars) CK(cudaMallocHost(reinterpret_cast<void**>(&m->h_scalars), 64 * 3 * sizeof(int)));
  int* slot = m->h_scalars + 3 * (m->scalar_slot++ & 63);
  slot[0] = m->valid_len; slot[1] = m->valid_len - 1; slot[2] = m->n_ids;
  CK(cudaMemcpyAsync(m->d_valid_len, slot, 3 * sizeof(int), cudaMemcpyHostToDevice, st));
  return VLA_OK;
}

int vla_set_prompt_ids(vla_handle m, const int32_t* ids, int len, void* stream) {
  if (!m) return VLA_ERR_STATE;
  cudaSetDevice(m->cfg.device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (!m->embed_table) return m->fail(VLA_ERR_STATE, "vla_set_prompt_ids needs 'embedding_weight' loaded before vla_finalize");
  if (len < 0 || len > m->L) return m->fail(VLA_ERR_SHAPE, "prompt of %d tokens does not fit the window of %d", len, m->L);
  if (!m->pi05 && len != m->L) return m->fail(VLA_ERR_SHAPE, "Pi0 prompt length is fixed at %d", m->L);
  if (len > 0 && !ids) return m->fail(VLA_ERR_STATE, "null token ids");
  if (len > 0) CK(cudaMemcpyAsync(m->d_ids, ids, (size_t)len * sizeof(int32_t), cudaMemcpyDefault, st));
  m->n_ids = len;
  m->valid_len = m->nv * 256 + len;
  return upload_scalars(m, st);
}

int vla_set_prompt(vla_handle m, const void* embeds, int len, void* stream) {
  if (!m) return VLA_ERR_STATE;
  cudaSetDevice(m->cfg.device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (len < 0 || len > m->L) return m->fail(VLA_ERR_SHAPE, "prompt of %d rows does not fit the window of %d", len, m->L);
  if (!m->pi05 && len != m->L) return m->fail(VLA_ERR_SHAPE, "Pi0 prompt length is fixed at %d", m->L);
  CK(cudaMemsetAsync(m->lang, 0, (size_t)std::max(m->L, 1) * 2048 * 2, st));
  if (len > 0) CK(cudaMemcpyAsync(m->lang, embeds, (size_t)len * 2048 * 2, cudaMemcpyDefault, st));
  m->n_ids = -1;     // the prompt rows are embeddings: the id gather inside the graph stays idle
  m->valid_len = m->nv * 256 + len;
  return upload_scalars(m, st);
}

int vla_finalize(vla_handle m) {
  if (!m) return VLA_ERR_STATE;
  if (m->finalized) return m->fail(VLA_ERR_STATE, "already finalized");
  cudaSetDevice(m->cfg.device);
  // RoPE tables, theta 10000, fp32 (pi0_infer.py:1319-1335)
  {
    const int n_pos = m->T + 1;
    std::vector<float> c((size_t)n_pos * 128), s((size_t)n_pos * 128);
    for (int i = 0; i < 128; ++i) {
      const float inv_freq = 1.0f / std::pow(10000.0f, (float)(2 * i) / 256.0f);
      for (int pos = 0; pos < n_pos; ++pos) {
        const float ph = inv_freq * (float)pos;
        c[(size_t)pos * 128 + i] = (float)std::cos((double)ph);
        s[(size_t)pos * 128 + i] = (float)std::sin((double)ph);
      }
    }
    CK(cudaMemcpy(m->rope_cos, c.data(), c.size() * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(m->rope_sin, s.data(), s.size() * 4, cudaMemcpyHostToDevice));
  }
  int rc = upload_scalars(m, m->own_stream);
  if (rc) return rc;
  CK(cudaStreamSynchronize(m->own_stream));
  if (m->pi05) {
    if (m->named.find("decoder_time_embeds") == m->named.end()) {
      bf16* dst = nullptr;
      if (!m->dalloc(&dst, (size_t)10 * 1024, "decoder_time_embeds")) return m->fail(VLA_ERR_CUDA, "allocation failed");
    }
    rc = pi05_precompute(m, m->own_stream);
    if (rc) return rc;
  }
  if (m->use_xp) {
    rc = xp_pack(m);
    if (rc) return rc;
  }
  Plan pl{m};
  plan_vision(pl);
  plan_prefix(pl);
  plan_decoder(pl);
  if (!pl.ok) return m->fail(VLA_ERR_CUDA, "plan: %s", pl.err.c_str());
  // one eager run (sets function attributes, surfaces launch errors), then capture (pi0_infer.py:1347-1354)
  rc = run_ops(m, m->own_stream);
  if (rc) return rc;
  CK(cudaStreamSynchronize(m->own_stream));
  rc = check_status(m);
  if (rc) return rc;
  if (m->use_graph) {
    CK(cudaStreamBeginCapture(m->own_stream, cudaStreamCaptureModeThreadLocal));
    rc = run_ops(m, m->own_stream);
    cudaError_t ce = cudaStreamEndCapture(m->own_stream, &m->graph);
    if (rc) return rc;
    if (ce != cudaSuccess) return m->fail(VLA_ERR_CUDA, "graph capture failed: %s", cudaGetErrorString(ce));
    CK(cudaGraphInstantiate(&m->graph_exec, m->graph, 0));
  }
  m->finalized = true;
  return VLA_OK;
}

int vla_buffer(vla_handle m, const char* name, void** dev_ptr, size_t* bytes) {
  if (!m || !name) return VLA_ERR_STATE;
  auto it = m->named.find(name);
  if (it == m->named.end()) return m->fail(VLA_ERR_KEY, "unknown buffer '%s'", name);
  if (dev_ptr) *dev_ptr = it->second.first;
  if (bytes) *bytes = it->second.second;
  return VLA_OK;
}

int vla_forward(vla_handle m, void* stream) {
  if (!m || !m->finalized) return m ? m->fail(VLA_ERR_STATE, "forward before finalize") : VLA_ERR_STATE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  cudaSetDevice(m->cfg.device);
  if (m->use_graph) {
    CK(cudaGraphLaunch(m->graph_exec, st));
    return VLA_OK;
  }
  return run_ops(m, st);
}

int vla_forward_stages(vla_handle m, int stage_mask, void* stream) {
  if (!m || !m->finalized) return m ? m->fail(VLA_ERR_STATE, "forward before finalize") : VLA_ERR_STATE;
  if (stage_mask <= 0 || stage_mask > 7) return m->fail(VLA_ERR_SHAPE, "stage mask must be a combination of 1 (vision), 2 (prefix), 4 (action expert)");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  cudaSetDevice(m->cfg.device);
  if (stage_mask == 7) return vla_forward(m, stream);
  if (!m->use_graph) {
    for (int sidx = 0; sidx < 3; ++sidx)
      if (stage_mask & (1 << sidx)) { int rc = run_ops(m, st, sidx); if (rc) return rc; }
    return VLA_OK;
  }
  auto it = m->stage_graphs.find(stage_mask);
  if (it == m->stage_graphs.end()) {
    cudaGraph_t g = nullptr;
    CK(cudaStreamSynchronize(m->own_stream));
    CK(cudaStreamBeginCapture(m->own_stream, cudaStreamCaptureModeThreadLocal));
    int rc = VLA_OK;
    for (int sidx = 0; sidx < 3 && !rc; ++sidx)
      if (stage_mask & (1 << sidx)) rc = run_ops(m, m->own_stream, sidx);
    cudaError_t ce = cudaStreamEndCapture(m->own_stream, &g);
    if (rc) return rc;
    if (ce != cudaSuccess) return m->fail(VLA_ERR_CUDA, "stage graph capture failed: %s", cudaGetErrorString(ce));
    cudaGraphExec_t ge = nullptr;
    CK(cudaGraphInstantiate(&ge, g, 0));
    cudaGraphDestroy(g);
    it = m->stage_graphs.emplace(stage_mask, ge).first;
  }
  CK(cudaGraphLaunch(it->second, st));
  return VLA_OK;
}

// ---- multi-view latency mode: image tokens pushed over NVLink inside the captured graphs (link.cuh) -----------------
namespace {
void drop_stage_graphs(vla_model* m) {
  for (auto& kv : m->stage_graphs) cudaGraphExecDestroy(kv.second);
  m->stage_graphs.clear();
}
int link_export(vla_model* m, unsigned char* ipc_handle_out, void** local_ptr_out) {
  if (ipc_handle_out) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the header promises 64 bytes");
    cudaIpcMemHandle_t h;
    CK(cudaIpcGetMemHandle(&h, m->link_box));
    memcpy(ipc_handle_out, &h, sizeof h);
  }
  if (local_ptr_out) *local_ptr_out = m->link_box;
  return VLA_OK;
}
}  // namespace

int vla_link_trunk_create(vla_handle m, int n_views, unsigned char* ipc_handle_out, void** local_ptr_out) {
  if (!m || !m->finalized) return m ? m->fail(VLA_ERR_STATE, "link before finalize") : VLA_ERR_STATE;
  if (m->link_box) return m->fail(VLA_ERR_STATE, "this handle already has a mailbox");
  if (m->B != 1 || n_views < 1 || n_views > lk::MAX_VIEWS || n_views != m->nv)
    return m->fail(VLA_ERR_SHAPE, "the trunk of latency mode is a single-observation handle with one tower per view (%d views)", m->nv);
  cudaSetDevice(m->cfg.device);
  const size_t bytes = lk::TRUNK_STAGING_OFF + (size_t)2 * n_views * lk::TILE_FLOATS * sizeof(float);
  if (!m->dalloc(&m->link_box, bytes)) return m->fail(VLA_ERR_CUDA, "mailbox allocation failed");
  m->link_views = n_views;
  // the towers check the view count they were given against this word
  CK(cudaMemcpy(m->link_box + lk::TRUNK_VIEWS * sizeof(unsigned int), &n_views, sizeof(int), cudaMemcpyHostToDevice));
  return link_export(m, ipc_handle_out, local_ptr_out);
}

int vla_link_tower_create(vla_handle m, unsigned char* ipc_handle_out, void** local_ptr_out) {
  if (!m || !m->finalized) return m ? m->fail(VLA_ERR_STATE, "link before finalize") : VLA_ERR_STATE;
  if (m->link_box) return m->fail(VLA_ERR_STATE, "this handle already has a mailbox");
  if (m->B != 1 || m->nv != 1) return m->fail(VLA_ERR_SHAPE, "a tower of latency mode is a single-observation, single-view handle");
  cudaSetDevice(m->cfg.device);
  if (!m->dalloc(&m->link_box, lk::TOWER_BOX_BYTES)) return m->fail(VLA_ERR_CUDA, "mailbox allocation failed");
  m->link_views = 0;
  return link_export(m, ipc_handle_out, local_ptr_out);
}

int vla_link_open(vla_handle m, const unsigned char* ipc_handle, void** ptr_out) {
  if (!m || !ipc_handle || !ptr_out) return VLA_ERR_STATE;
  cudaSetDevice(m->cfg.device);
  cudaIpcMemHandle_t h;
  memcpy(&h, ipc_handle, sizeof h);
  void* p = nullptr;
  CK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  m->ipc_opened.push_back(p);
  *ptr_out = p;
  return VLA_OK;
}

int vla_link_tower_connect(vla_handle m, void* trunk_mailbox, int view, int n_views) {
  if (!m || !m->link_box || m->link_views != 0 || !trunk_mailbox) return m ? m->fail(VLA_ERR_STATE, "not a tower with a mailbox") : VLA_ERR_STATE;
  if (m->link_connected) return m->fail(VLA_ERR_STATE, "tower already connected");
  if (view < 0 || view >= n_views || n_views > lk::MAX_VIEWS) return m->fail(VLA_ERR_SHAPE, "view %d of %d", view, n_views);
  cudaSetDevice(m->cfg.device);
  {
    int trunk_views = 0;   // the staging slots are laid out for the trunk's view count
    CK(cudaMemcpy(&trunk_views, reinterpret_cast<const unsigned int*>(trunk_mailbox) + lk::TRUNK_VIEWS, sizeof(int), cudaMemcpyDeviceToHost));
    if (trunk_views != n_views) return m->fail(VLA_ERR_SHAPE, "the trunk's mailbox was created for %d views, this tower was given %d", trunk_views, n_views);
  }
  const float4* tile = reinterpret_cast<const float4*>(m->encoder_x);
  float4* staging = reinterpret_cast<float4*>(reinterpret_cast<uint8_t*>(trunk_mailbox) + lk::TRUNK_STAGING_OFF);
  unsigned int* flags = reinterpret_cast<unsigned int*>(trunk_mailbox);
  unsigned int* box = reinterpret_cast<unsigned int*>(m->link_box);
  int* status = m->d_status;
  const int grid = m->sm_count;
  // last node of the vision stage
  auto it = m->ops.begin();
  for (auto j = m->ops.begin(); j != m->ops.end(); ++j)
    if (j->stage == 0) it = j + 1;
  m->ops.insert(it, {0, true, [=](cudaStream_t st) {
                       lk::push_kernel<<<grid, 256, 0, st>>>(tile, staging, flags, box, view, n_views, status);
                       return cudaGetLastError();
                     }});
  m->n_kernels++;
  m->link_connected = true;
  drop_stage_graphs(m);
  return VLA_OK;
}

int vla_link_trunk_connect(vla_handle m, int view, void* tower_mailbox) {
  if (!m || !m->link_box || m->link_views == 0 || !tower_mailbox) return m ? m->fail(VLA_ERR_STATE, "not a trunk with a mailbox") : VLA_ERR_STATE;
  if (view < 0 || view >= m->link_views) return m->fail(VLA_ERR_SHAPE, "view %d of %d", view, m->link_views);
  cudaSetDevice(m->cfg.device);
  unsigned int* ack = reinterpret_cast<unsigned int*>(tower_mailbox) + lk::TOWER_ACK;
  CK(cudaMemcpy(m->link_box + lk::TRUNK_ACK_OFF + view * sizeof(unsigned int*), &ack, sizeof ack, cudaMemcpyHostToDevice));
  if (!m->link_connected) {
    float4* x = reinterpret_cast<float4*>(m->encoder_x);
    unsigned int* box = reinterpret_cast<unsigned int*>(m->link_box);
    const int n_views = m->link_views, grid = m->sm_count;
    int* status = m->d_status;
    // first node of the prefix stage
    auto it = m->ops.begin();
    while (it != m->ops.end() && it->stage < 1) ++it;
    m->ops.insert(it, {1, true, [=](cudaStream_t st) {
                         lk::wait_kernel<<<grid, 256, 0, st>>>(x, box, n_views, status);
                         return cudaGetLastError();
                       }});
    m->n_kernels++;
    m->link_connected = true;
    drop_stage_graphs(m);
  }
  return VLA_OK;
}

int vla_forward_host(vla_handle m, const void* images, const void* state, const void* noise, void* actions_out) {
  if (!m || !m->finalized) return m ? m->fail(VLA_ERR_STATE, "forward before finalize") : VLA_ERR_STATE;
  if (!images || !noise || !actions_out || (!m->pi05 && !state)) return m->fail(VLA_ERR_STATE, "null input");
  cudaSetDevice(m->cfg.device);
  cudaStream_t st = m->own_stream;
  const size_t B = m->B;
  CK(cudaMemcpyAsync(m->images, images, B * m->nv * 224 * 224 * 3 * 2, cudaMemcpyHostToDevice, st));
  if (!m->pi05) CK(cudaMemcpyAsync(m->state, state, B * 32 * 2, cudaMemcpyHostToDevice, st));
  CK(cudaMemcpyAsync(m->noise, noise, B * m->C * 32 * 2, cudaMemcpyHostToDevice, st));
  int rc = vla_forward(m, st);
  if (rc) return rc;
  CK(cudaMemcpyAsync(actions_out, m->noise, B * m->C * 32 * 2, cudaMemcpyDeviceToHost, st));
  // the status word rides along: a bounded wait that ran out or a clamped token id must not pass silently
  if (!m->h_status) CK(cudaMallocHost(reinterpret_cast<void**>(&m->h_status), sizeof(int)));
  CK(cudaMemcpyAsync(m->h_status, m->d_status, sizeof(int), cudaMemcpyDeviceToHost, st));
  CK(cudaStreamSynchronize(st));
  if (*m->h_status) {
    const int w = *m->h_status;
    cudaMemsetAsync(m->d_status, 0, sizeof(int), st);
    return m->fail(VLA_ERR_DEVICE, "device status word 0x%x (bit 0: a bounded wait ran out, bit 1: bad shape / token id); cleared", w);
  }
  return VLA_OK;
}

// Pillow's precompute_coeffs + normalize_coeffs_8bpc for the BILINEAR filter over a whole axis, in the same
// double arithmetic (src/libImaging/Resample.c of Pillow; the reference resizes with Image.resize(..., BILINEAR),
// test.py:107).  Tables are built once per (input size, output size) and kept on the device.
static int resample_table(vla_model* m, int in_size, int out_size, vla_model::ResampleTable* out) {
  auto key = std::make_pair(in_size, out_size);
  auto it = m->resample.find(key);
  if (it != m->resample.end()) { *out = it->second; return VLA_OK; }
  const double scale = (double)in_size / (double)out_size;
  const double filterscale = scale < 1.0 ? 1.0 : scale;
  const double support = 1.0 * filterscale;
  const int ksize = (int)std::ceil(support) * 2 + 1;
  std::vector<int> bounds((size_t)out_size * 2), kk((size_t)out_size * ksize, 0);
  std::vector<double> w(ksize);
  const double ss = 1.0 / filterscale;
  for (int xx = 0; xx < out_size; ++xx) {
    const double center = (xx + 0.5) * scale;
    int xmin = (int)(center - support + 0.5);
    if (xmin < 0) xmin = 0;
    int xmax = (int)(center + support + 0.5);
    if (xmax > in_size) xmax = in_size;
    xmax -= xmin;
    double ww = 0.0;
    for (int x = 0; x < ksize; ++x) w[x] = 0.0;
    for (int x = 0; x < xmax; ++x) {
      double a = (x + xmin - center + 0.5) * ss;
      if (a < 0.0) a = -a;
      w[x] = a < 1.0 ? 1.0 - a : 0.0;
      ww += w[x];
    }
    for (int x = 0; x < xmax; ++x)
      if (ww != 0.0) w[x] /= ww;
    for (int x = 0; x < ksize; ++x)
      kk[(size_t)xx * ksize + x] = w[x] < 0 ? (int)(-0.5 + w[x] * (1 << PP_PRECISION_BITS)) : (int)(0.5 + w[x] * (1 << PP_PRECISION_BITS));
    bounds[2 * xx] = xmin;
    bounds[2 * xx + 1] = xmax;
  }
  vla_model::ResampleTable t{ksize, nullptr, nullptr};
  if (!m->dalloc(&t.bounds, bounds.size()) || !m->dalloc(&t.kk, kk.size())) return m->fail(VLA_ERR_CUDA, "allocation failed");
  CK(cudaMemcpy(t.bounds, bounds.data(), bounds.size() * sizeof(int), cudaMemcpyHostToDevice));
  CK(cudaMemcpy(t.kk, kk.data(), kk.size() * sizeof(int), cudaMemcpyHostToDevice));
  m->resample[key] = t;
  *out = t;
  return VLA_OK;
}

int vla_preprocess_image(vla_handle m, int obs, int view, const uint8_t* frame, int height, int width, void* stream) {
  if (!m || !m->finalized) return VLA_ERR_STATE;
  cudaSetDevice(m->cfg.device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (obs < 0 || obs >= m->B || view < 0 || view >= m->nv) return m->fail(VLA_ERR_SHAPE, "observation %d / view %d out of range", obs, view);
  if (!frame || height < 1 || width < 1 || height > 8192 || width > 8192) return m->fail(VLA_ERR_SHAPE, "frame must be (1..8192, 1..8192, 3) uint8");
  // sizes and paste offsets exactly as the host code computes them (test.py:99-113); a 224 x 224 frame passes through
  int rh = 224, rw = 224, pad_h = 0, pad_w = 0;
  if (!(width == 224 && height == 224)) {
    const double ratio = std::max((double)width / 224.0, (double)height / 224.0);
    rh = (int)((double)height / ratio);
    rw = (int)((double)width / ratio);
    pad_h = std::max(0, (int)((224 - rh) / 2.0));
    pad_w = std::max(0, (int)((224 - rw) / 2.0));
  }
  if (rh < 1 || rw < 1) return m->fail(VLA_ERR_SHAPE, "frame of %d x %d is too elongated to resize to 224 x 224", height, width);
  const size_t frame_bytes = (size_t)height * width * 3, tmp_bytes = (size_t)height * rw * 3;
  const size_t need = ((frame_bytes + 255) & ~(size_t)255) + tmp_bytes;
  if (need > m->pp_frame_cap) {   // grows only when a larger camera format shows up
    CK(cudaStreamSynchronize(st));
    uint8_t* q = nullptr;
    CK(cudaMalloc(&q, need));
    if (m->pp_frame) {
      for (auto& a : m->allocs)
        if (a == m->pp_frame) a = q;
      cudaFree(m->pp_frame);
    } else {
      m->allocs.push_back(q);
    }
    m->bytes += need - m->pp_frame_cap;
    m->pp_frame = q;
    m->pp_frame_cap = need;
  }
  vla_model::ResampleTable th, tv;
  int rc = resample_table(m, width, rw, &th);
  if (rc) return rc;
  rc = resample_table(m, height, rh, &tv);
  if (rc) return rc;
  uint8_t* tmp = m->pp_frame + ((frame_bytes + 255) & ~(size_t)255);
  // a frame that already lives on this GPU is read in place; anything else is staged first
  const uint8_t* src = frame;
  cudaPointerAttributes at;
  const bool on_device = cudaPointerGetAttributes(&at, frame) == cudaSuccess && at.type == cudaMemoryTypeDevice && at.device == m->cfg.device;
  (void)cudaGetLastError();   // an unregistered host pointer is not an error here
  if (!on_device) {
    CK(cudaMemcpyAsync(m->pp_frame, frame, frame_bytes, cudaMemcpyDefault, st));
    src = m->pp_frame;
  }
  pp_resize_h_kernel<<<(unsigned)((height * rw + 255) / 256), 256, 0, st>>>(src, height, width, tmp, rw, th.bounds, th.kk, th.ksize);
  bf16* dst = m->images + ((size_t)obs * m->nv + view) * 224 * 224 * 3;
  pp_resize_v_pad_norm_kernel<<<(224 * 224 + 255) / 256, 256, 0, st>>>(tmp, height, rw, rh, pad_h, pad_w, tv.bounds, tv.kk, tv.ksize, dst);
  CK(cudaGetLastError());
  return VLA_OK;
}

static int pp_small_buffers(vla_model* m) {
  if (!m->pp_vec && !m->dalloc(&m->pp_vec, 256)) return m->fail(VLA_ERR_CUDA, "allocation failed");
  if (!m->pp_out && !m->dalloc(&m->pp_out, (size_t)m->C * 32)) return m->fail(VLA_ERR_CUDA, "allocation failed");
  return VLA_OK;
}

int vla_preprocess_state(vla_handle m, int obs, const double* state, const double* a, const double* b, int n, int mode,
                         double* normalized_out, void* stream) {
  if (!m || !m->finalized) return VLA_ERR_STATE;
  cudaSetDevice(m->cfg.device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (obs < 0 || obs >= m->B || n < 1 || n > 32 || !state || !a || !b || (mode != 0 && mode != 1))
    return m->fail(VLA_ERR_SHAPE, "state: 1..32 values with two statistics vectors, mode 0 or 1");
  int rc = pp_small_buffers(m);
  if (rc) return rc;
  double host[96];
  for (int i = 0; i < n; ++i) { host[i] = state[i]; host[n + i] = a[i]; host[2 * n + i] = b[i]; }
  CK(cudaMemcpyAsync(m->pp_vec, host, (size_t)3 * n * sizeof(double), cudaMemcpyHostToDevice, st));
  // Pi05 has no state input buffer (its state goes into the prompt as tokens): only the float64 values come back
  bf16* dst = m->pi05 ? nullptr : m->state + (size_t)obs * 32;
  pp_state_kernel<<<1, 32, 0, st>>>(m->pp_vec, n, mode, dst, m->pp_vec + 128);
  CK(cudaGetLastError());
  if (normalized_out) {
    CK(cudaMemcpyAsync(normalized_out, m->pp_vec + 128, (size_t)n * sizeof(double), cudaMemcpyDefault, st));
    CK(cudaStreamSynchronize(st));
  }
  return VLA_OK;
}

int vla_postprocess_actions(vla_handle m, int obs, const double* a, const double* b, int n_stats, int mode,
                            const double* state_raw, int n_state, int action_dim, double* out, void* stream) {
  if (!m || !m->finalized) return VLA_ERR_STATE;
  cudaSetDevice(m->cfg.device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (obs < 0 || obs >= m->B || n_stats < 1 || n_stats > 32 || action_dim < 1 || action_dim > 32 || n_state < action_dim ||
      n_state > 32 || !a || !b || !state_raw || !out || (mode != 0 && mode != 1))
    return m->fail(VLA_ERR_SHAPE, "actions: 1..32 statistics, action_dim <= state length <= 32, mode 0 or 1");
  int rc = pp_small_buffers(m);
  if (rc) return rc;
  double host[96];
  for (int i = 0; i < n_stats; ++i) { host[i] = a[i]; host[n_stats + i] = b[i]; }
  for (int i = 0; i < n_state; ++i) host[2 * n_stats + i] = state_raw[i];
  CK(cudaMemcpyAsync(m->pp_vec, host, (size_t)(2 * n_stats + n_state) * sizeof(double), cudaMemcpyHostToDevice, st));
  const int total = m->C * action_dim;
  pp_actions_kernel<<<(total + 127) / 128, 128, 0, st>>>(m->noise + (size_t)obs * m->C * 32, m->C, m->pp_vec, n_stats, n_state, mode,
                                                          action_dim, m->pp_out);
  CK(cudaGetLastError());
  CK(cudaMemcpyAsync(out, m->pp_out, (size_t)total * sizeof(double), cudaMemcpyDefault, st));
  CK(cudaStreamSynchronize(st));
  return VLA_OK;
}

int vla_status_word(vla_handle m, int* out) {
  if (!m || !out) return VLA_ERR_STATE;
  cudaSetDevice(m->cfg.device);
  CK(cudaMemcpy(out, m->d_status, sizeof(int), cudaMemcpyDeviceToHost));
  return VLA_OK;
}

int vla_clear_status(vla_handle m) {
  if (!m) return VLA_ERR_STATE;
  cudaSetDevice(m->cfg.device);
  CK(cudaMemset(m->d_status, 0, sizeof(int)));
  return VLA_OK;
}

int vla_stats(vla_handle m, int* n_kernels, size_t* device_bytes) {
  if (!m) return VLA_ERR_STATE;
  if (n_kernels) *n_kernels = m->n_kernels;
  if (device_bytes) *device_bytes = m->bytes;
  return VLA_OK;
}

int vla_stage_kernels(vla_handle m, int* n3) {
  if (!m || !m->finalized || !n3) return VLA_ERR_STATE;
  n3[0] = n3[1] = n3[2] = 0;
  for (const auto& op : m->ops)
    if (op.is_kernel && op.stage >= 0 && op.stage < 3) n3[op.stage]++;
  return VLA_OK;
}

int vla_time_stages(vla_handle m, float* ms3) {
  if (!m || !m->finalized || !ms3) return VLA_ERR_STATE;
  cudaSetDevice(m->cfg.device);
  cudaEvent_t ev[4];
  for (auto& e : ev) CK(cudaEventCreate(&e));
  cudaStream_t st = m->own_stream;
  CK(cudaEventRecord(ev[0], st));
  for (int s = 0; s < 3; ++s) {
    int rc = run_ops(m, st, s);
    if (rc) return rc;
    CK(cudaEventRecord(ev[s + 1], st));
  }
  CK(cudaStreamSynchronize(st));
  for (int s = 0; s < 3; ++s) CK(cudaEventElapsedTime(&ms3[s], ev[s], ev[s + 1]));
  for (auto& e : ev) cudaEventDestroy(e);
  return VLA_OK;
}

int vla_destroy(vla_handle m) {
  if (!m) return VLA_OK;
  cudaSetDevice(m->cfg.device);
  cudaDeviceSynchronize();
  if (m->graph_exec) cudaGraphExecDestroy(m->graph_exec);
  for (auto& kv : m->stage_graphs) cudaGraphExecDestroy(kv.second);
  if (m->graph) cudaGraphDestroy(m->graph);
  if (m->own_stream) cudaStreamDestroy(m->own_stream);
  if (m->h_scalars) cudaFreeHost(m->h_scalars);
  if (m->h_status) cudaFreeHost(m->h_status);
  for (void* p : m->ipc_opened) cudaIpcCloseMemHandle(p);
  for (void* p : m->allocs) cudaFree(p);
  delete m;
  return VLA_OK;
}

// ---- single operators ------------------------------------------------------------------------------
#define CKG(call)                                                                  \
  do {                                                                             \
    cudaError_t e_ = (call);                                                       \
    if (e_ != cudaSuccess) {                                                       \
      g_last_error = std::string(#call) + " failed: " + cudaGetErrorString(e_);    \
      rc = VLA_ERR_CUDA;                                                           \
      goto done;                                                                   \
    }                                                                              \
  } while (0)

int vla_op_gemm(const vla_gemm_desc* d, void* stream) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int rc = VLA_OK;
  bf16 *wt = nullptr, *wt2 = nullptr;
  float *cosT = nullptr, *sinT = nullptr, *scratch = nullptr;
  int* status = nullptr;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  const int Kp = round_up(d->K, 64), Np = round_up(d->N, 128);
  int dev = 0, sms = 148;
  GemmOp op;
  GemmEpi e;
  std::string err;
  memset(&e, 0, sizeof e);
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  CKG(cudaMalloc(&wt, (size_t)Np * Kp * 2));
  CKG(cudaMalloc(&status, 4));
  CKG(cudaMemsetAsync(status, 0, 4, st));
  {
    dim3 grid((Np + 31) / 32, (Kp + 31) / 32), block(32, 8);
    repack_kn_to_nk<<<grid, block, 0, st>>>(reinterpret_cast<const bf16*>(d->w), d->K, d->N, wt, Kp, Np);
    if (d->w2) {
      CKG(cudaMalloc(&wt2, (size_t)Np * Kp * 2));
      repack_kn_to_nk<<<grid, block, 0, st>>>(reinterpret_cast<const bf16*>(d->w2), d->K, d->N, wt2, Kp, Np);
    }
  }
  e.kind = d->epi; e.act = d->act; e.bias = d->bias;
  e.out = reinterpret_cast<bf16*>(d->out_bf16); e.ld_out = d->ld_out > 0 ? d->ld_out : d->N;
  e.outf = d->out_f32; e.ld_outf = d->N; e.res_in = d->res; e.res_mod = d->res_mod; e.ld_res = d->N; e.gate = d->gate;
  if (d->epi == EPI_QKV) {
    if (d->N != 2560) { g_last_error = "QKV epilogue needs N = 2560"; rc = VLA_ERR_SHAPE; goto done; }
    const int n_pos = d->pos_off + d->rows_per_obs + 1;
    std::vector<float> c((size_t)n_pos * 128), s((size_t)n_pos * 128);
    for (int i = 0; i < 128; ++i) {
      const float inv_freq = 1.0f / std::pow(10000.0f, (float)(2 * i) / 256.0f);
      for (int pos = 0; pos < n_pos; ++pos) {
        c[(size_t)pos * 128 + i] = (float)std::cos((double)(inv_freq * (float)pos));
        s[(size_t)pos * 128 + i] = (float)std::sin((double)(inv_freq * (float)pos));
      }
    }
    CKG(cudaMalloc(&cosT, c.size() * 4));
    CKG(cudaMalloc(&sinT, s.size() * 4));
    CKG(cudaMemcpy(cosT, c.data(), c.size() * 4, cudaMemcpyHostToDevice));
    CKG(cudaMemcpy(sinT, s.data(), s.size() * 4, cudaMemcpyHostToDevice));
    e.q = reinterpret_cast<bf16*>(d->q); e.kc = reinterpret_cast<bf16*>(d->kcache); e.vc = reinterpret_cast<bf16*>(d->vcache);
    e.rope_cos = cosT; e.rope_sin = sinT; e.pos_off = d->pos_off; e.rows_per_obs = d->rows_per_obs;
    e.kv_obs_stride = d->kv_obs_stride; e.kv_row_off = d->kv_row_off;
    e.vt = reinterpret_cast<bf16*>(d->vt); e.vt_ld = d->vt_ld;
  }
  if (!build_gemm(&op, wt, wt2, d->N, Np, Kp, reinterpret_cast<const bf16*>(d->x), d->tokens, d->K, d->K, e, status, sms,
                  d->bn, d->split, &err, d->pair == 2 ? -1 : d->pair, d->tok_tile, d->pair == 2 ? 1 : (d->pair == 0 ? 0 : -1))) {
    g_last_error = err;
    rc = VLA_ERR_SHAPE;
    goto done;
  }
  if (gemm_scratch_floats(op.bn, op.dual, op.grid, op.p.cg2) > 0) {
    CKG(cudaMalloc(&scratch, gemm_scratch_floats(op.bn, op.dual, op.grid, op.p.cg2) * sizeof(float)));
    op.p.scratch = scratch;
  }
  CKG(launch_gemm(op, st, false));
  CKG(cudaStreamSynchronize(st));
  if (d->iters > 0 && d->ms_per_iter) {
    // timing loop: only meaningful for epilogues that are idempotent (not the in-place residual)
    CKG(cudaEventCreate(&e0));
    CKG(cudaEventCreate(&e1));
    CKG(cudaEventRecord(e0, st));
    for (int i = 0; i < d->iters; ++i) CKG(launch_gemm(op, st, false));
    CKG(cudaEventRecord(e1, st));
    CKG(cudaStreamSynchronize(st));
    float ms = 0.f;
    CKG(cudaEventElapsedTime(&ms, e0, e1));
    *d->ms_per_iter = ms / d->iters;
  }
  {
    int w = 0;
    CKG(cudaMemcpy(&w, status, 4, cudaMemcpyDeviceToHost));
    if (w) { g_last_error = "device status word raised: bounded wait timed out"; rc = VLA_ERR_DEVICE; }
  }
done:
  if (e0) cudaEventDestroy(e0);
  if (e1) cudaEventDestroy(e1);
  cudaFree(wt); cudaFree(wt2); cudaFree(cosT); cudaFree(sinT); cudaFree(status); cudaFree(scratch);
  return rc;
}

int vla_op_attention(const vla_attn_desc* d, void* stream) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int rc = VLA_OK;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  float* scratch = nullptr;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (d->head_dim != 72 && d->head_dim != 256) { g_last_error = "head_dim must be 72 or 256"; return VLA_ERR_SHAPE; }
  AttnParams a;
  memset(&a, 0, sizeof a);
  a.q = reinterpret_cast<const bf16*>(d->q); a.k = reinterpret_cast<const bf16*>(d->k);
  a.v = reinterpret_cast<const bf16*>(d->v); a.o = reinterpret_cast<bf16*>(d->o);
  a.ldq = d->ldq; a.ldk = d->ldk; a.ldv = d->ldv; a.ldo = d->ldo;
  a.q_go = d->q_go; a.q_gi = d->q_gi; a.k_go = d->k_go; a.k_gi = d->k_gi; a.v_go = d->v_go; a.v_gi = d->v_gi; a.o_go = d->o_go; a.o_gi = d->o_gi;
  a.g_inner = d->groups_inner; a.n_q = d->n_q; a.n_keys = d->n_keys;
  a.prefix_alloc = d->prefix_alloc; a.valid_prefix = d->valid_prefix; a.restrict_rows = d->restrict_rows;
  a.scale_log2e = d->scale * 1.4426950408889634f;
  const int groups = d->groups_outer * d->groups_inner;
  a.ksplit = d->ksplit > 0 ? d->ksplit : pick_ksplit(d->n_q, d->n_keys, groups, sms);
  if (a.ksplit > 8 || (a.ksplit & (a.ksplit - 1))) { g_last_error = "ksplit must be 1, 2, 4 or 8"; return VLA_ERR_SHAPE; }
  if (a.ksplit > 1) {
    CKG(cudaMalloc(&scratch, attn_scratch_floats(a, d->head_dim, groups) * sizeof(float)));
    a.scratch = scratch;
  }
  CKG(launch_attn(a, d->head_dim, groups, st, false));
  CKG(cudaStreamSynchronize(st));
  if (d->iters > 0 && d->ms_per_iter) {
    CKG(cudaEventCreate(&e0));
    CKG(cudaEventCreate(&e1));
    CKG(cudaEventRecord(e0, st));
    for (int i = 0; i < d->iters; ++i) CKG(launch_attn(a, d->head_dim, groups, st, false));
    CKG(cudaEventRecord(e1, st));
    CKG(cudaStreamSynchronize(st));
    float ms = 0.f;
    CKG(cudaEventElapsedTime(&ms, e0, e1));
    *d->ms_per_iter = ms / d->iters;
  }
done:
  if (e0) cudaEventDestroy(e0);
  if (e1) cudaEventDestroy(e1);
  cudaFree(scratch);
  return rc;
}

// ---- allocation-free GEMM -----------------------------------------------------------------------------
// Scratch for the split-K partial tiles of vla_op_gemm_noalloc: part of the library image, so it exists on
// every GPU that loads the library from load time until exit and no call ever has to allocate it.
#define VLA_NOALLOC_SCRATCH_FLOATS (1u << 20)   /* 4 MiB */
static __device__ __align__(256) float vla_noalloc_scratch[VLA_NOALLOC_SCRATCH_FLOATS];
// Status word of the same entry point (a bounded wait inside the kernel that ran out sets bit 0): also part of the
// library image, so reporting a timeout needs no allocation either.
static __device__ int vla_noalloc_status;

int vla_op_vit_attention_tc(const void* qkv, void* o, int views, float scale, int iters, float* ms_per_iter, void* stream) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int rc = VLA_OK;
  int* status = nullptr;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  VitAttnTcParams p;
  if (!qkv || !o || views < 1) { g_last_error = "vla_op_vit_attention_tc: bad arguments"; return VLA_ERR_SHAPE; }
  CKG(cudaMalloc(&status, sizeof(int)));
  CKG(cudaMemsetAsync(status, 0, sizeof(int), st));
  p.qkv = reinterpret_cast<const bf16*>(qkv); p.o = reinterpret_cast<bf16*>(o);
  p.scale_log2e = scale * 1.4426950408889634f; p.status = status; p.trace = nullptr;
  CKG(launch_vit_attn_tc(p, views, st, false));
  if (iters > 0 && ms_per_iter) {
    CKG(cudaEventCreate(&e0));
    CKG(cudaEventCreate(&e1));
    CKG(cudaEventRecord(e0, st));
    for (int i = 0; i < iters; ++i) CKG(launch_vit_attn_tc(p, views, st, false));
    CKG(cudaEventRecord(e1, st));
    CKG(cudaEventSynchronize(e1));
    float ms = 0.f;
    CKG(cudaEventElapsedTime(&ms, e0, e1));
    *ms_per_iter = ms / iters;
  }
  CKG(cudaStreamSynchronize(st));
  {
    int h = 0;
    CKG(cudaMemcpy(&h, status, sizeof(int), cudaMemcpyDeviceToHost));
    if (h) { g_last_error = "vla_op_vit_attention_tc: device status word raised"; rc = VLA_ERR_DEVICE; }
  }
done:
  if (e0) cudaEventDestroy(e0);
  if (e1) cudaEventDestroy(e1);
  if (status) cudaFree(status);
  return rc;
}

// per-device addresses of the two symbols above, looked up on the first call on that device
struct NoallocDev { float* scratch = nullptr; int* status = nullptr; };
static NoallocDev* noalloc_device(int* dev_out) {
  // In host code the arrays' names are only handles for the runtime, not device addresses, so they must go through
  // cudaGetSymbolAddress with the target device current; the result differs per device.
  static NoallocDev table[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { g_last_error = "vla_op_gemm_noalloc: no current device"; return nullptr; }
  NoallocDev& nd = table[dev];
  if (!nd.scratch) {
    float* ptr = nullptr;
    int* sptr = nullptr;
    cudaError_t ce = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), vla_noalloc_scratch);
    if (ce == cudaSuccess) ce = cudaGetSymbolAddress(reinterpret_cast<void**>(&sptr), vla_noalloc_status);
    if (ce != cudaSuccess || !ptr || !sptr) {
      g_last_error = std::string("vla_op_gemm_noalloc: cudaGetSymbolAddress failed: ") + cudaGetErrorString(ce);
      return nullptr;
    }
    nd.status = sptr;
    nd.scratch = ptr;
  }
  if (dev_out) *dev_out = dev;
  return &nd;
}

int vla_op_gemm_noalloc(const vla_gemm_noalloc_desc* d, void* stream) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (!d || !d->x || !d->w_nk || !d->out_bf16) { g_last_error = "vla_op_gemm_noalloc: null argument"; return VLA_ERR_STATE; }
  int dev = 0, sms = 148;
  NoallocDev* nd = noalloc_device(&dev);
  if (!nd) return VLA_ERR_CUDA;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (d->K % 8) { g_last_error = "vla_op_gemm_noalloc: K must be a multiple of 8 (16-byte rows for TMA)"; return VLA_ERR_SHAPE; }
  if (d->k_pad % 64 || d->n_pad % 128 || d->k_pad < d->K || d->n_pad < d->N) {
    g_last_error = "vla_op_gemm_noalloc: w_nk must be [n_pad, k_pad] with n_pad % 128 == 0, k_pad % 64 == 0, covering N x K";
    return VLA_ERR_SHAPE;
  }
  GemmEpi e;
  memset(&e, 0, sizeof e);
  e.kind = EPI_BF16;
  e.act = ACT_NONE;
  e.bias = d->bias;
  e.out = reinterpret_cast<bf16*>(d->out_bf16);
  e.ld_out = d->N;
  GemmOp op;
  std::string err;
  // split = 0: take the library's choice, then halve it until the partial tiles fit the built-in array (an unsplit
  // launch needs none); an explicit split that does not fit is the caller's error
  int split = d->split;
  for (;;) {
    if (!build_gemm(&op, reinterpret_cast<const bf16*>(d->w_nk), nullptr, d->N, d->n_pad, d->k_pad,
                    reinterpret_cast<const bf16*>(d->x), d->tokens, d->K, d->K, e, nd->status, sms, 0, split, &err, -1, 0, -1, false)) {
      g_last_error = "vla_op_gemm_noalloc: " + err;
      return VLA_ERR_SHAPE;
    }
    if (gemm_scratch_floats(op.bn, op.dual, op.grid, op.p.cg2) <= VLA_NOALLOC_SCRATCH_FLOATS) break;
    if (d->split != 0 || op.p.split <= 1) {
      char buf[200];
      snprintf(buf, sizeof buf, "vla_op_gemm_noalloc: this shape needs %zu scratch floats, the built-in scratch holds %u; "
               "use a smaller split or vla_op_gemm", gemm_scratch_floats(op.bn, op.dual, op.grid, op.p.cg2), VLA_NOALLOC_SCRATCH_FLOATS);
      g_last_error = buf;
      return VLA_ERR_LIMIT;
    }
    split = op.p.split / 2;
  }
  op.p.scratch = nd->scratch;
  cudaError_t ce = launch_gemm(op, st, false);
  if (ce != cudaSuccess) { g_last_error = std::string("vla_op_gemm_noalloc: launch failed: ") + cudaGetErrorString(ce); return VLA_ERR_CUDA; }
  return VLA_OK;
}

int vla_op_gemm_noalloc_status(int* out) {
  if (!out) return VLA_ERR_STATE;
  NoallocDev* nd = noalloc_device(nullptr);
  if (!nd) return VLA_ERR_CUDA;
  int zero = 0;
  // both copies synchronise with the device; neither allocates
  if (cudaMemcpy(out, nd->status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess ||
      cudaMemcpy(nd->status, &zero, sizeof(int), cudaMemcpyHostToDevice) != cudaSuccess) {
    g_last_error = std::string("vla_op_gemm_noalloc_status: ") + cudaGetErrorString(cudaGetLastError());
    return VLA_ERR_CUDA;
  }
  return VLA_OK;
}

// Timeline of the persistent action-expert kernel: one run of the expert stage on the handle's own stream with
// CTA 0 recording %globaltimer at every grid barrier (arrival, release).  out[2 i], out[2 i + 1] in nanoseconds.
int vla_expert_timeline(vla_handle m, unsigned long long* out, int max_entries, int* n_written) {
  if (!m || !m->finalized || !out || !n_written) return VLA_ERR_STATE;
  if (!m->use_xp) return m->fail(VLA_ERR_STATE, "the persistent action-expert kernel is not in use for this handle");
  cudaSetDevice(m->cfg.device);
  const int phases = m->nsteps * ((m->pi05 ? 1 : 2) + 6 * m->nl + 1);
#ifdef XP_FINE_TRACE
  const int n = std::min(4096, max_entries);   // development build: the in-phase marks sit behind the barrier records
#else
  const int n = std::min(std::min(2 * phases, 4096), max_entries);
#endif
  CK(cudaMemsetAsync(m->xp_trace, 0, 4096 * sizeof(unsigned long long), m->own_stream));
  CK(launch_expert_persistent(m, m->own_stream, m->xp_trace));
  CK(cudaStreamSynchronize(m->own_stream));
  CK(cudaMemcpy(out, m->xp_trace, (size_t)n * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
  *n_written = n;
  return VLA_OK;
}

int vla_op_attention_tc(const vla_attn_tc_desc* d, void* stream) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int rc = VLA_OK;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  float* scratch = nullptr;
  int* status = nullptr;
  int dev = 0, sms = 148;
  AttnTcOp op;
  std::string err;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int ks = d->ksplit > 0 ? d->ksplit : pick_ksplit_tc(d->n_q, d->n_keys, sms);
  if (ks > 8 || (ks & (ks - 1))) { g_last_error = "ksplit must be 1, 2, 4 or 8"; return VLA_ERR_SHAPE; }
  CKG(cudaMalloc(&status, 4));
  CKG(cudaMemsetAsync(status, 0, 4, st));
  if (ks > 1) CKG(cudaMalloc(&scratch, attn_tc_scratch_floats(d->n_q, ks) * sizeof(float)));
  if (!build_attn_tc(&op, reinterpret_cast<const bf16*>(d->q), reinterpret_cast<const bf16*>(d->k), d->k_rows,
                     reinterpret_cast<const bf16*>(d->vt), d->vt_ld, reinterpret_cast<bf16*>(d->o), 256, d->n_q, d->n_keys,
                     d->prefix_alloc, d->valid_prefix, nullptr, d->restrict_rows, d->scale, ks, scratch, status, &err)) {
    g_last_error = err;
    rc = VLA_ERR_SHAPE;
    goto done;
  }
  CKG(launch_attn_tc(op, st, false));
  CKG(cudaStreamSynchronize(st));
  if (d->iters > 0 && d->ms_per_iter) {
    CKG(cudaEventCreate(&e0));
    CKG(cudaEventCreate(&e1));
    CKG(cudaEventRecord(e0, st));
    for (int i = 0; i < d->iters; ++i) CKG(launch_attn_tc(op, st, false));
    CKG(cudaEventRecord(e1, st));
    CKG(cudaStreamSynchronize(st));
    float ms = 0.f;
    CKG(cudaEventElapsedTime(&ms, e0, e1));
    *d->ms_per_iter = ms / d->iters;
  }
  {
    int w = 0;
    CKG(cudaMemcpy(&w, status, 4, cudaMemcpyDeviceToHost));
    if (w) { g_last_error = "device status word raised: bounded wait timed out"; rc = VLA_ERR_DEVICE; }
  }
done:
  if (e0) cudaEventDestroy(e0);
  if (e1) cudaEventDestroy(e1);
  cudaFree(scratch);
  cudaFree(status);
  return rc;
}

int vla_op_norm(const float* x, void* y, int rows, int D, int mode, const float* w, const float* b, void* stream) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  cudaError_t e = launch_norm(x, D, reinterpret_cast<bf16*>(y), D, rows, D, mode, w, b, 0, 0, 0, st, false);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) { g_last_error = std::string("norm failed: ") + cudaGetErrorString(e); return VLA_ERR_CUDA; }
  return VLA_OK;
}

}  // extern "C"
