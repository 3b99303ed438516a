// libflyb200: host side of the C ABI declared in include/flyb200.h — argument
// checks, tensor-map encoding, kernel selection and launch.  No allocation, no
// synchronisation and no memcpy on the launch path.
#include "../../include/flyb200.h"
#include "launch.h"
#include "quant_kernel.cuh"

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

using namespace flyb200;
using flyb200::host::MAX_DEVICES;
using flyb200::host::SMEM_LIMIT;
using flyb200::host::ROWS2_STAGES;

namespace {

thread_local char g_cuda_err[256] = "";

int cuda_fail(cudaError_t e, const char* what) {
  snprintf(g_cuda_err, sizeof(g_cuda_err), "%s: %s", what, cudaGetErrorString(e));
  return FLYB200_E_CUDA;
}
#define CUDA_TRY(expr)                                   \
  do {                                                   \
    cudaError_t _e = (expr);                             \
    if (_e != cudaSuccess) return cuda_fail(_e, #expr);  \
  } while (0)

// Device status word: kernels record the first failed bounded wait here.
__device__ int g_status_word = 0;

struct DeviceState {
  std::once_flag once;
  int sms = 0;
  int* status = nullptr;
  cudaError_t err = cudaSuccess;
};
DeviceState g_dev[MAX_DEVICES];

int device_state(DeviceState** out) {
  int dev = 0;
  CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= MAX_DEVICES) return FLYB200_E_UNSUPPORTED;
  DeviceState& st = g_dev[dev];
  std::call_once(st.once, [&]() {
    st.err = cudaDeviceGetAttribute(&st.sms, cudaDevAttrMultiProcessorCount, dev);
    if (st.err == cudaSuccess) st.err = cudaGetSymbolAddress(reinterpret_cast<void**>(&st.status), g_status_word);
  });
  if (st.err != cudaSuccess) return cuda_fail(st.err, "device setup");
  *out = &st;
  return FLYB200_OK;
}

// cuTensorMapEncodeTiled through the runtime's driver entry point lookup, so
// the library does not link libcuda.
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// 2-D row-major byte/half matrix, 128-byte swizzled boxes.
int make_map(CUtensorMap* m, CUtensorMapDataType dt, int elem_bytes, const void* base, uint64_t inner_elems,
             uint64_t rows, uint32_t box_inner_elems, uint32_t box_rows) {
  EncodeTiledFn enc = get_encode();
  if (!enc) {
    snprintf(g_cuda_err, sizeof(g_cuda_err), "cuTensorMapEncodeTiled entry point not found");
    return FLYB200_E_CUDA;
  }
  cuuint64_t dims[2] = {inner_elems, rows};
  cuuint64_t strides[1] = {inner_elems * static_cast<uint64_t>(elem_bytes)};
  cuuint32_t box[2] = {box_inner_elems, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(g_cuda_err, sizeof(g_cuda_err), "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
    return FLYB200_E_CUDA;
  }
  return FLYB200_OK;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline int kind_of(int in_dtype) {
  return in_dtype == FLYB200_DT_FP8 ? KIND_F8 : in_dtype == FLYB200_DT_INT8 ? KIND_I8 : in_dtype == FLYB200_DT_FP16 ? KIND_F16 : KIND_BF16;
}
inline int elem_bytes_of(int in_dtype) { return (in_dtype == FLYB200_DT_FP8 || in_dtype == FLYB200_DT_INT8) ? 1 : 2; }

constexpr size_t TICKET_BYTES = 16384;  // 4096 channel tiles
constexpr int MAX_SPLIT_K = 32;

// The preshuffled weights as a 3-D tensor {128 bytes, N rows, K/128 k-blocks}; boxes of
// 128 rows x one k-block are copied verbatim (the image is already swizzled).
int make_weight_map(CUtensorMap* m, const void* base, uint64_t n_rows, uint64_t k_blocks, uint32_t box_rows) {
  EncodeTiledFn enc = get_encode();
  if (!enc) {
    snprintf(g_cuda_err, sizeof(g_cuda_err), "cuTensorMapEncodeTiled entry point not found");
    return FLYB200_E_CUDA;
  }
  cuuint64_t dims[3] = {KBLOCK_BYTES, n_rows, k_blocks};
  cuuint64_t strides[2] = {KBLOCK_BYTES, n_rows * KBLOCK_BYTES};
  cuuint32_t box[3] = {KBLOCK_BYTES, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(g_cuda_err, sizeof(g_cuda_err), "cuTensorMapEncodeTiled (weights) failed with CUresult %d",
             static_cast<int>(r));
    return FLYB200_E_CUDA;
  }
  return FLYB200_OK;
}

// Output window [rows, cols] of a wider row-major matrix (row pitch given in
// elements), 2-byte elements, 64 x 32 boxes with the 128-byte swizzle.
int make_window_map(CUtensorMap* m, CUtensorMapDataType dt, const void* base, uint64_t cols, uint64_t rows,
                    uint64_t pitch_elems) {
  EncodeTiledFn enc = get_encode();
  if (!enc) {
    snprintf(g_cuda_err, sizeof(g_cuda_err), "cuTensorMapEncodeTiled entry point not found");
    return FLYB200_E_CUDA;
  }
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {pitch_elems * 2};
  cuuint32_t box[2] = {64, 32};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(g_cuda_err, sizeof(g_cuda_err), "cuTensorMapEncodeTiled (output window) failed with CUresult %d",
             static_cast<int>(r));
    return FLYB200_E_CUDA;
  }
  return FLYB200_OK;
}

// Ring depth of the small-M kernel: as deep as ~200 KB of shared memory allow, at most 12.
inline int default_decode_stages(int bn, int w_rows = BLOCK_ROWS) {
  if (w_rows == BLOCK_ROWS) return bn <= 64 ? 8 : (bn <= 128 ? 6 : 4);
  const int stage = (w_rows + bn) * KBLOCK_BYTES;
  int n = 200 * 1024 / stage;
  return n > 12 ? 12 : (n < 2 ? 2 : n);
}

// Ring depth of the pair form (a stage is 16 KiB of weights + bn / 2 tokens).
inline int default_decode2_stages(int bn) { return bn <= 128 ? 8 : 6; }

inline int decode_bn_for(int M) { return M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256; }

// Split-K factor that simply covers the SMs, with at least four k-blocks per
// CTA (the built-in-scratch entry point sizes its split with this).
// `token_blocks`: CTAs per channel tile that the token split already provides.
int fill_sms_split_k(int N, int K_bytes, int sms, int token_blocks = 1) {
  const int n_tiles = ((N + BLOCK_ROWS - 1) / BLOCK_ROWS) * token_blocks;
  const int kb = K_bytes / KBLOCK_BYTES;
  if (n_tiles >= sms || n_tiles > static_cast<int>(TICKET_BYTES / sizeof(int))) return 1;
  int split = sms / n_tiles;
  if (split > kb / 4) split = kb / 4;
  if (split > MAX_SPLIT_K) split = MAX_SPLIT_K;
  return split < 1 ? 1 : split;
}

// Estimated time (ns) of the small-M kernel for a split-K factor, from rates
// measured on B200 (N = K = 8192 and 4096, 1..256 tokens):
//   fixed      ~3 us: launch, first bytes from DRAM, exit.
//   stream     a CTA takes in ~71 B/ns (its 16 KiB weight block from DRAM plus the
//              token tile from L2 share the SM's input port); all CTAs together
//              cannot beat a read-only stream over the GPU (~7 TB/s).  CTAs
//              beyond one per SM run in a second round.
//   reduction  cluster: two cluster barriers and a remote round trip (~1.5 us)
//              plus the (split-1)/split of a partial tile (bn x 512 B) every CTA
//              reads from its peers at ~15 B/ns; clusters of more than four CTAs
//              measured ~10 us slower than the model when they cover more than
//              half of the SMs (scheduling of large clusters that each need a
//              whole SM's shared memory; eight clusters of eight are fine: 16 x
//              1024 x 8192 5.7 us, 32 x 1024 x 28672 11.1 us).  Workspace: ~3 us
//              (ticket, fences) plus the last CTA reading `split` partial tiles
//              from L2, latency-bound at ~14 B/ns (16 x 1024 x 8192 with 13
//              splits: 12.4 us), so it is what remains when a cluster cannot
//              supply enough CTAs.
// Reproduces the measured ranking: split 2 at 64 channel tiles (14.5 us against
// 21 us unsplit and 15 us for split 4), split 4 at 32 tiles of 128 tokens (9.8 us
// against 12.1 / 19.0 / 21.4 us for 2 / 1 / 8).
// `pair`: CTA pairs, each CTA stages half of the tokens and the cluster is twice the split.
double split_cost_ns(int split, int n_tiles, int kb, int bn, int sms, bool cluster, bool pair = false) {
  const double stage_bytes = static_cast<double>(BLOCK_ROWS * KBLOCK_BYTES + (pair ? bn / 2 : bn) * KBLOCK_BYTES);
  const int rounds = (n_tiles * split + sms - 1) / sms;
  const int kbs = (kb + split - 1) / split;
  double stream = rounds * kbs * stage_bytes / 71.0;
  const double hbm = static_cast<double>(n_tiles) * kb * (BLOCK_ROWS * KBLOCK_BYTES) / 7000.0;
  if (stream < hbm) stream = hbm;
  double reduce = 0.0;
  if (split > 1) {
    const double partial = bn * 512.0;
    // Clusters have to be placed whole inside a GPC, so fewer CTAs are resident at once than there are
    // SMs: clusters of more than four CTAs are slow to place when they cover more than two thirds of
    // the SMs (16 x 8 CTAs: 12.2 us against 7.3 us for 16 x 4; 12 x 8 is fine), clusters of three or
    // more when they cover more than 90 % (48 x 3 = 144 CTAs: 18.3 us against 12.0 us for 48 x 2).
    const int csize = pair ? 2 * split : split;
    const bool crowded = (csize > 4 && 3 * n_tiles * split > 2 * sms) || (csize >= 3 && 10 * n_tiles * split > 9 * sms);
    reduce = cluster ? 1500.0 + (split - 1.0) / split * partial / 15.0 + (crowded ? 10000.0 : 0.0)
                     : 3000.0 + split * partial / 14.0;
  }
  return 3000.0 + stream + reduce;
}

// Split-K factor of the small-M kernel when the caller does not force one: the
// cheapest by split_cost_ns over cluster splits 1..8 and, where a workspace of
// the needed size was passed, workspace splits 9..32.  Every split keeps at
// least two k-blocks per CTA.
int auto_split_k(int N, int K_bytes, int sms, int bn, int token_blocks, size_t workspace_bytes, bool have_ws,
                 bool pair = false, double* cost_out = nullptr) {
  const int n_tiles = ((N + BLOCK_ROWS - 1) / BLOCK_ROWS) * token_blocks;
  const int kb = K_bytes / KBLOCK_BYTES;
  int best = 1;
  double best_cost = split_cost_ns(1, n_tiles, kb, bn, sms, true, pair);
  // Only splits that keep the launch within one round of CTAs: with more CTAs than SMs the
  // later rounds wait for whole CTAs to retire (measured at 64 tiles, K = 28672, 64 tokens:
  // split 9 = four rounds 77 us, split 2 = one round 40 us, where the model's rates said 9).
  for (int s = 2; n_tiles * s <= sms && s <= MAX_SPLIT_K && 2 * s <= kb; ++s) {
    if (pair && 2 * s > MAX_CLUSTER_SPLIT) break;  // pairs combine their K splits inside one cluster only
    const bool cluster = s <= MAX_CLUSTER_SPLIT;
    if (!cluster) {
      if (!have_ws || n_tiles > static_cast<int>(TICKET_BYTES / sizeof(int))) break;
      const size_t need = TICKET_BYTES + static_cast<size_t>(s) * n_tiles * bn * BLOCK_ROWS * sizeof(uint32_t);
      if (workspace_bytes < need) break;
    }
    const double c = split_cost_ns(s, n_tiles, kb, bn, sms, cluster, pair);
    if (c < best_cost) {
      best_cost = c;
      best = s;
    }
  }
  if (cost_out) *cost_out = best_cost;
  return best;
}

size_t partial_bytes(int split, int N, int bn, int token_blocks = 1) {
  const size_t n_tiles = static_cast<size_t>((N + BLOCK_ROWS - 1) / BLOCK_ROWS) * token_blocks;
  return static_cast<size_t>(split) * n_tiles * bn * BLOCK_ROWS * sizeof(uint32_t);
}

struct Plan {
  bool decode;
  bool two_sm;  // large-M kernel as CTA pairs (tcgen05 cta_group::2)
  bool tall;    // large-M kernel with 256-row tiles (two accumulators per CTA)
  int token_blocks;  // small-M kernel: the tokens are split into this many blocks of bn (grid.z)
  int w_rows;        // small-M kernel: output channels per CTA (128, or 64 without any K split)
  bool pair;         // small-M kernel as CTA pairs (256 channels per pair, half of the tokens staged per CTA)
  int bn;
  int split_k;
  int kb_per_split;
  int group_m;
  int reduce_mode;
  int stages;
  int pdl;
  int prefetch;  // k-blocks of weights requested into L2 ahead of the ring
};

// 0 = off, 1 = on, 2 = on and the weights are known to be static
int pdl_default() {
  static const int mode = []() {
    const char* e = getenv("FLYB200_PDL");
    if (!e) return 1;
    return e[0] == '1' ? 1 : e[0] == '2' ? 2 : 0;
  }();
  return mode;
}

// FLYB200_PREFETCH_DECODE: tuning override of the small-M kernel's prefetch distance (k-blocks); -1 = not set
int decode_prefetch_override() {
  static const int n = []() {
    const char* e = getenv("FLYB200_PREFETCH_DECODE");
    if (!e) return -1;
    const int v = atoi(e);
    return v < 0 ? 0 : v;
  }();
  return n;
}

bool w64_default() {
  static const bool on = []() {
    // Off unless asked for: with one CTA streaming a tile's whole K range the
    // single MMA-issuing thread (about 290 cycles per k-block) becomes the limit;
    // measured 21 us against 14.5 us for 128-channel tiles with split-K 2
    // (M = 32, N = K = 8192).
    const char* e = getenv("FLYB200_DECODE_W64");
    return e && e[0] == '1';
  }();
  return on;
}

// FLYB200_DECODE_PAIR=1: CTA pairs wherever the small-M kernel has more than 32 tokens.  Off unless asked
// for (also per call: kernel field 5 of the hint): each CTA then takes in a third fewer bytes, but a
// k-block is consumed only once both CTAs hold their halves and freed by a commit that has to reach the
// peer, and graph-replayed launches measured within -5 % .. +4 % of the one-CTA form (FP8, N = K = 8192,
// 256 tokens: 25.4 against 24.4 us; K = 28672: 55.0 against 56.9 us; N = 16384: 42.3 against 44.5 us).
bool decode_pair_default() {
  static const bool on = []() {
    const char* e = getenv("FLYB200_DECODE_PAIR");
    return e && e[0] == '1';
  }();
  return on;
}

// FLYB200_ROWS_TALL=1: 256-row tiles for the large-M kernel wherever no other form is asked for
bool rows_tall_default() {
  static const bool on = []() {
    const char* e = getenv("FLYB200_ROWS_TALL");
    return e && e[0] == '1';
  }();
  return on;
}

bool rows_two_sm_default() {
  static const bool on = []() {
    const char* e = getenv("FLYB200_ROWS_2SM");
    return e && e[0] == '1';
  }();
  return on;
}

// variant_hint fields (see include/flyb200.h)
inline int hint_split(int h) { return h & 0xFF; }
inline int hint_kernel(int h) { return (h >> 8) & 0xF; }
inline int hint_reduce(int h) { return (h >> 12) & 0xF; }
inline int hint_group(int h) { return (h >> 16) & 0xFF; }
inline int hint_stages(int h) { return (h >> 24) & 0xF; }
inline int hint_pdl(int h) { return (h >> 28) & 0x3; }
inline int hint_tokens(int h) { return (h >> 30) & 0x3; }

bool workspace_fits(bool have_ws, size_t ws_bytes, int split, int N, int bn, int token_blocks) {
  return have_ws && ws_bytes >= TICKET_BYTES + partial_bytes(split, N, bn, token_blocks) &&
         ((N + BLOCK_ROWS - 1) / BLOCK_ROWS) * token_blocks <= static_cast<int>(TICKET_BYTES / sizeof(int));
}

// How many blocks the tokens of the small-M kernel are split into when the
// caller does not say.  Splitting the tokens gives more CTAs per channel tile
// without a reduction step, but every weight block is then fetched once per
// token block; measured on B200 (N = K = 8192, M = 32..256) that costs more
// than the split-K reduction it saves (21 us vs 14.5 us at M = 32), so the
// automatic choice is one block and the split stays a tuning option.
int auto_token_blocks(int /*M*/, int /*N*/, int /*sms*/) { return 1; }

// Tile width of the large-M kernel when the caller does not force one.  All
// tiles are 128 tokens high; the kernel is persistent, so a launch takes
// ceil(tiles / SMs) rounds of one tile per SM.  Per 128-byte k-block a tile
// costs the largest of: the tensor pipe (2 * bn cycles), the single thread
// that issues the MMAs (ROWS_ISSUE_CYCLES), and bringing the operands into
// shared memory ((16 KiB + bn * 128 B) / ROWS_LOAD_BYTES_PER_CYCLE).  The
// width with the cheapest whole launch wins; ties go to the wider tile (fewer
// operand bytes per flop).
constexpr int ROWS_ISSUE_CYCLES = 300;
constexpr int ROWS_LOAD_BYTES_PER_CYCLE = 96;
constexpr int ROWS_TILE_OVERHEAD_CYCLES = 2000;  // pipeline fill and the last, exposed epilogue of a CTA
int auto_rows_bn(int M, int N, int K_bytes, int sms) {
  const long long num_m = (M + BLOCK_ROWS - 1) / BLOCK_ROWS;
  const long long kb = K_bytes / KBLOCK_BYTES;
  long long best_cost = -1;
  int best = 256;
  for (int bn = 256; bn >= 64; bn -= 32) {
    const long long tiles = num_m * ((N + bn - 1) / bn);
    const long long rounds = (tiles + sms - 1) / sms;
    long long per_kb = 2 * bn;
    if (per_kb < ROWS_ISSUE_CYCLES) per_kb = ROWS_ISSUE_CYCLES;
    const long long load = (BLOCK_ROWS * KBLOCK_BYTES + bn * KBLOCK_BYTES) / ROWS_LOAD_BYTES_PER_CYCLE;
    if (per_kb < load) per_kb = load;
    const long long cost = rounds * (kb * per_kb + 4 * bn) + ROWS_TILE_OVERHEAD_CYCLES;
    if (best_cost < 0 || cost < best_cost) {
      best_cost = cost;
      best = bn;
    }
  }
  return best;
}

// `allow_pair`: the caller's kind has the CTA-pair form of the small-M kernel (the plain kinds do)
int make_plan(Plan* plan, int M, int N, int K_bytes, int variant_hint, size_t workspace_bytes, bool have_ws, int sms,
              bool allow_pair = true) {
  const int want_kernel = hint_kernel(variant_hint);
  const int want_split = hint_split(variant_hint);
  const int want_reduce = hint_reduce(variant_hint);
  if (want_kernel > 6) return FLYB200_E_BAD_ARG;
  plan->decode = (want_kernel == 1 || want_kernel == 4 || want_kernel == 5) ? true : want_kernel >= 2 ? false : (M <= 256);
  if (want_kernel == 0 && plan->decode) {
    // Wide outputs: the small-M kernel launches one CTA per 128 channels, so with more channel
    // tiles than SMs it runs in rounds and the last one is part empty; the large-M kernel is
    // persistent and walks 256-channel tiles.  Measured (FP8, K = 8192, us, small-M / large-M):
    // N = 28672 (224 tiles): M = 32 47/48, 64 49/49, 96 55/49, 200 71/66; N = 24576 (192 tiles, the
    // second round 30 % full): M = 16 43/41, 32 46/41, 64 48/41, 96 53/42; N = 57344 (448 tiles):
    // M = 16 89/81, 32 95/83, 96 104/85; N = 18944 (exactly one round): M = 96 31/32, 200 41/43.
    const int tiles = (N + BLOCK_ROWS - 1) / BLOCK_ROWS;
    const int rounds = (tiles + sms - 1) / sms;
    const bool poor_fill = 10 * tiles < 7 * rounds * sms;  // the rounds are less than 70 % full
    // (16 tokens on a very wide output: 89/81 at K = 8192, but 52/62 at K = 4096)
    const bool very_wide = tiles >= 3 * sms && (M > 16 || (M == 16 && K_bytes >= 8192));
    if (tiles > sms && (M > 64 || (poor_fill && M >= 32) || very_wide)) plan->decode = false;
  }
  if (want_kernel == 0 && M > 256 && M <= 1024) {
    // Narrow outputs with 257..1024 tokens and a long K: the large-M kernel has too few tiles for the
    // SMs and no K split; the small-M kernel takes the tokens in blocks of 256 (grid.z) and splits K
    // over a cluster.  Taken where (channel tiles x token blocks) leave room for a split of two or
    // more in one round of CTAs.  Measured, small-M / large-M, us: 512 x 2048 x 8192 16.3 / 23.5,
    // 512 x 4096 x 8192 24.1 / 26.5, 1024 x 2048 x 8192 24.1 / 26.9; with 128 unsplit CTAs the
    // large-M kernel wins (512 x 8192 x 8192 41.9 / 38.5).
    const int ctas = ((N + BLOCK_ROWS - 1) / BLOCK_ROWS) * ((M + 255) / 256);
    plan->decode = 2 * ctas <= sms && K_bytes / KBLOCK_BYTES >= 32;
  }
  plan->two_sm = want_kernel == 3 ? true : (want_kernel == 2 || want_kernel == 6) ? false : rows_two_sm_default();
  plan->tall = !plan->decode && !plan->two_sm && (want_kernel == 6 || (want_kernel == 0 && rows_tall_default()));
  if (want_kernel == 0 && !plan->decode && !plan->two_sm && !plan->tall && want_split == 0) {
    // 256-row tiles where they cover the output in ONE nearly full round of CTAs: every SM then does
    // the flops of two 128-row tiles but fetches its weight blocks once (1024 x 8192 x 8192: 59-60 us
    // against 62-65 us).  With more rounds the 128-row form wins: it overlaps the epilogue of a
    // tile with the mainloop of the next, which the 256-row form (all of TMEM in one tile) cannot.
    // (Not where the taller tiles would add a padded half tile of rows, nor for M <= 256.)
    const long long t = static_cast<long long>((M + 255) / 256) * ((N + 255) / 256);
    const bool no_extra_rows = (M + 255) / 256 * 2 == (M + 127) / 128;
    plan->tall = M > 256 && no_extra_rows && t <= sms && 5 * t >= 4 * sms;
  }
  if (plan->decode && M > 1024) return FLYB200_E_UNSUPPORTED;  // up to four token blocks of 256
  if (want_reduce > REDUCE_CLUSTER) return FLYB200_E_BAD_ARG;
  plan->token_blocks = 1;
  plan->w_rows = BLOCK_ROWS;
  plan->pair = false;
  if (!plan->decode) {
    // large-M kernel: the split field carries the tile width in units of 32 channels
    if (plan->two_sm) {
      plan->bn = 256;
    } else if (want_split > 0) {
      if (want_split > 8) return FLYB200_E_BAD_ARG;
      plan->bn = 32 * want_split;
    } else if (plan->tall) {
      plan->bn = 256;
    } else {
      plan->bn = auto_rows_bn(M, N, K_bytes, sms);
    }
  }
  if (plan->decode) {
    const int ht = hint_tokens(variant_hint);
    int t = ht == 0 ? auto_token_blocks(M, N, sms) : (ht == 1 ? 1 : ht == 2 ? 2 : 4);
    plan->bn = decode_bn_for((M + t - 1) / t);
    plan->token_blocks = (M + plan->bn - 1) / plan->bn;  // no empty block
    // CTA pairs: from 64-token tiles up, where the token tile is a large part of what an SM takes in
    const int tiles = (N + BLOCK_ROWS - 1) / BLOCK_ROWS;
    const bool pair_ok = plan->bn >= 64 && (tiles & 1) == 0 && want_reduce != REDUCE_WORKSPACE && want_split <= MAX_CLUSTER_SPLIT / 2;
    if (want_kernel == 5 && !pair_ok) return FLYB200_E_UNSUPPORTED;
    plan->pair = pair_ok && (want_kernel == 5 || (want_kernel == 0 && allow_pair && decode_pair_default()));
  }
  // 32 row tiles (32 MiB of 8-bit activations at K = 8192) stay in L2 while a group walks the channels:
  // measured DRAM reads 1.17 x the operands against 1.67 x with groups of 16, at equal time
  plan->group_m = hint_group(variant_hint) > 0 ? hint_group(variant_hint) : (plan->two_sm ? 8 : plan->tall ? 16 : 32);
  plan->split_k = 1;
  plan->reduce_mode = REDUCE_NONE;
  if (plan->decode) {
    // 64-channel tiles: when they alone put one CTA on (nearly) every SM, no K
    // split and therefore no reduction step is needed.
    const int tiles64 = (N + 63) / 64;
    const bool fits = plan->bn <= 64 && plan->token_blocks == 1 && !plan->pair;
    const bool wanted = want_kernel == 4;
    const bool automatic = want_kernel == 0 && want_split == 0 && want_reduce == 0 && tiles64 <= sms &&
                           4 * tiles64 >= 3 * sms && w64_default();
    if (wanted && (!fits || want_split > 1 || want_reduce != 0)) return FLYB200_E_UNSUPPORTED;
    if (fits && (wanted || automatic)) plan->w_rows = 64;
  }
  plan->stages = hint_stages(variant_hint) >= 2 ? hint_stages(variant_hint)
                 : plan->pair                   ? default_decode2_stages(plan->bn)
                                                : default_decode_stages(plan->bn, plan->w_rows);
  // The two MMA issuers take alternate k-blocks.  With an even ring depth a stage
  // always belongs to the same issuer, so its full-barrier is never more than
  // one phase ahead of the thread waiting on it (a parity wait cannot tell
  // phase n from phase n + 2).  An odd depth becomes the next even one, or the
  // one below when that does not fit into shared memory.
  if (plan->stages & 1) {
    const int deeper = plan->pair ? decode2_layout(plan->bn, plan->stages + 1).total
                                  : decode_layout(plan->bn, plan->stages + 1, plan->w_rows).total;
    plan->stages += deeper <= SMEM_LIMIT ? 1 : -1;
  }
  // Weights requested into L2 ahead of the ring.  Small-M kernel: four k-blocks
  // beyond the depth of the ring measured best (INT8 32 x 8192 x 8192 on one GPU:
  // 13.9 us with 12 blocks ahead of an 8-deep ring, 14.4 us with 8, 14.7 us with
  // none, 15.3 us with the whole K range requested at once).  Large-M kernel:
  // none; there the weights of a tile are shared by the CTAs of a group and
  // mostly hit L2 already, and the extra requests cost 1-30 %.
  plan->prefetch = 0;  // small-M kernel: set below, once the ring depth is known
  if (plan->decode) plan->prefetch = decode_prefetch_override() >= 0 ? decode_prefetch_override() : plan->stages + 4;
  const int hp = hint_pdl(variant_hint);
  plan->pdl = hp == 1 ? 1 : hp == 2 ? 0 : hp == 3 ? 2 : pdl_default();
  if (!plan->decode) {
    // Large-M kernels: programmatic dependent launch only for launches of at most two rounds of tiles,
    // where hiding the launch and set-up behind the previous kernel's tail is worth 2-6 % (512 x 4096 x
    // 4096: 18.0 -> 16.9 us); on long launches it measured 0.5 % slower.  The CTA-pair form runs without it.
    const long long rows = plan->tall ? 2 * BLOCK_ROWS : BLOCK_ROWS;
    const long long tiles = ((M + rows - 1) / rows) * ((N + plan->bn - 1) / plan->bn);
    if (plan->two_sm || tiles > 2LL * sms) plan->pdl = 0;
  }
  const int kb = K_bytes / KBLOCK_BYTES;
  plan->kb_per_split = kb;
  if (plan->decode) {
    // (more than 256 tokens: cluster splits only, so that no such call ever needs a workspace)
    int split = want_split > 0 ? want_split
                               : auto_split_k(N, K_bytes, sms, plan->bn, plan->token_blocks, workspace_bytes,
                                              have_ws && M <= 256, plan->pair);
    if (plan->w_rows == 64) split = 1;
    if (split > kb) split = kb;
    int mode = REDUCE_NONE;
    if (split > 1) {
      mode = want_reduce != 0 ? want_reduce : (split <= MAX_CLUSTER_SPLIT ? REDUCE_CLUSTER : REDUCE_WORKSPACE);
      if (mode == REDUCE_CLUSTER && split > MAX_CLUSTER_SPLIT) {
        if (want_split > 0) return FLYB200_E_UNSUPPORTED;
        split = MAX_CLUSTER_SPLIT;
      }
      if (mode == REDUCE_WORKSPACE &&
          !workspace_fits(have_ws, workspace_bytes, split, N, plan->bn, plan->token_blocks)) {
        if (want_split > 0 || want_reduce != 0) return FLYB200_E_WORKSPACE;  // explicit requests are not changed silently
        split = split < MAX_CLUSTER_SPLIT ? split : MAX_CLUSTER_SPLIT;
        mode = REDUCE_CLUSTER;
      }
    }
    plan->kb_per_split = (kb + split - 1) / split;
    plan->split_k = (kb + plan->kb_per_split - 1) / plan->kb_per_split;
    plan->reduce_mode = plan->split_k > 1 ? mode : REDUCE_NONE;
  }
  return FLYB200_OK;
}

int gemm_common(void* c, const void* a, const void* w, const float* sa, const float* sb, const void* bias, int M,
                int N, int K, int in_dtype, int outmode, int epilogue, int variant_hint, void* workspace,
                size_t workspace_bytes, void* stream) {
  if (!c || !a || !w || M < 0 || N <= 0 || K <= 0) return FLYB200_E_BAD_ARG;
  if (in_dtype < FLYB200_DT_FP8 || in_dtype > FLYB200_DT_BF16) return FLYB200_E_BAD_ARG;
  if (epilogue < FLYB200_EPI_NONE || epilogue > FLYB200_EPI_BIAS_GELU) return FLYB200_E_BAD_ARG;
  if (epilogue != FLYB200_EPI_NONE && !bias) return FLYB200_E_BAD_ARG;
  const int eb = elem_bytes_of(in_dtype);
  if (eb == 1 && outmode != OUT_RAW32 && ((sa == nullptr) != (sb == nullptr))) return FLYB200_E_BAD_ARG;
  if (!flyb200_layout_kind(N, K, eb)) return FLYB200_E_UNSUPPORTED;
  if (!aligned16(c) || !aligned16(a) || !aligned16(w)) return FLYB200_E_BAD_ALIGN;
  if (workspace && !aligned16(workspace)) return FLYB200_E_BAD_ALIGN;
  if (M == 0) return FLYB200_OK;
  if (in_dtype == FLYB200_DT_FP16 || in_dtype == FLYB200_DT_BF16) {
    if (outmode == OUT_RAW32) return FLYB200_E_UNSUPPORTED;
  }

  DeviceState* st = nullptr;
  int rc = device_state(&st);
  if (rc) return rc;
  const int K_bytes = K * eb;

  Plan plan;
  rc = make_plan(&plan, M, N, K_bytes, variant_hint, workspace_bytes, workspace != nullptr, st->sms);
  if (rc) return rc;

  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.w = static_cast<const uint8_t*>(w);
  p.sa = sa;
  p.sb = sb;
  p.bias = bias;
  p.c = c;
  p.M = M;
  p.N = N;
  p.K_bytes = K_bytes;
  p.epilogue = epilogue;
  p.group_m = plan.group_m;
  p.split_k = plan.split_k;
  p.kb_per_split = plan.kb_per_split;
  p.reduce_mode = plan.reduce_mode;
  p.stages = plan.stages;
  p.pdl = plan.pdl;
  p.prefetch = plan.prefetch;
  p.token_blocks = plan.token_blocks;
  p.bn = plan.bn;
  p.rows_stages = plan.tall ? host::ROWS_TALL_STAGES : host::rows_stages_for(plan.bn);
  p.ws_tickets = static_cast<int*>(workspace);
  p.ws_partials = workspace ? reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + TICKET_BYTES) : nullptr;
  p.status = st->status;

  CUtensorMap tmA, tmC, tmW;
  memset(&tmC, 0, sizeof(tmC));
  memset(&tmW, 0, sizeof(tmW));
  if (!plan.decode && plan.two_sm) {
    rc = make_weight_map(&tmW, w, static_cast<uint64_t>(N), static_cast<uint64_t>(K_bytes / KBLOCK_BYTES), BLOCK_ROWS);
    if (rc) return rc;
  }
  rc = make_map(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a, static_cast<uint64_t>(K_bytes), static_cast<uint64_t>(M),
                KBLOCK_BYTES, plan.decode ? (plan.pair ? plan.bn / 2 : plan.bn) : plan.tall ? 2 * BLOCK_ROWS : BLOCK_ROWS);
  if (rc) return rc;
  if (!plan.decode && outmode != OUT_RAW32) {
    rc = make_map(&tmC, outmode == OUT_FP16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, c,
                  static_cast<uint64_t>(N), static_cast<uint64_t>(M), 64, 32);
    if (rc) return rc;
  }

  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int kind = kind_of(in_dtype);
  if (plan.decode && plan.pair) return host::launch_decode2_kind(kind, outmode, plan.bn, tmA, p, s);
  if (plan.decode) return host::launch_decode_kind(kind, outmode, plan.bn, plan.w_rows, tmA, p, s);
  const int form = plan.two_sm ? host::ROWS_FORM_PAIRS : plan.tall ? host::ROWS_FORM_TALL : host::ROWS_FORM_ONE;
  return host::launch_rows_kind(kind, outmode, form, tmA, tmW, tmC, p, st->sms, s);
}

// ---------------------------------------------------------------------------
// weight preshuffle: a pure byte permutation in 16-byte chunks
// ---------------------------------------------------------------------------
// chunk (row n, k-block blk, chunk c of 8) of the row-major matrix
//   row-major source offset : n*Kb + blk*128 + c*16
//   MFMA 16x16 source offset: ((n/16)*(Kb/16) + blk*8 + c)*256 + (n%16)*16
//   B200 image offset       : ((blk*N + n)*8 + (c ^ (n&7)))*16
template <int SRC_LAYOUT, bool INVERSE>
__global__ void shuffle_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, int N, int Kb) {
  const size_t total = static_cast<size_t>(N) * (Kb / 16);
  for (size_t g = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; g < total;
       g += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(g & 7);
    const size_t rest = g >> 3;
    const int n = static_cast<int>(rest % N);
    const size_t blk = rest / N;
    const size_t img = (blk * N + n) * 8 + (c ^ (n & 7));
    size_t plain;
    if (SRC_LAYOUT == FLYB200_SRC_ROW_MAJOR) {
      plain = (static_cast<size_t>(n) * Kb + blk * 128) / 16 + c;
    } else {
      plain = ((static_cast<size_t>(n >> 4) * (Kb / 16) + blk * 8 + c) * 256 + (n & 15) * 16) / 16;
    }
    if (INVERSE) {
      dst[plain] = src[img];
    } else {
      dst[img] = src[plain];
    }
  }
}

template <int SRC_LAYOUT, bool INVERSE>
int launch_shuffle(void* dst, const void* src, int N, int Kb, cudaStream_t s) {
  const size_t total = static_cast<size_t>(N) * (Kb / 16);
  const int threads = 256;
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 32) blocks = 148 * 32;
  shuffle_kernel<SRC_LAYOUT, INVERSE>
      <<<static_cast<unsigned>(blocks), threads, 0, s>>>(static_cast<uint4*>(dst), static_cast<const uint4*>(src), N, Kb);
  CUDA_TRY(cudaGetLastError());
  return FLYB200_OK;
}

// Row quantiser launch: rows that fit the register-cached single-pass kernel
// use it (one block per row), longer rows take the two-pass kernel.
template <typename TIn, bool FP8>
void launch_quant_t(uint8_t* y, float* scale, const TIn* x, int rows, int K, cudaStream_t s) {
  constexpr int per_vec = 256 * QuantIn<TIn>::VEC;
  if (K <= per_vec) {
    pertoken_quant_row_kernel<TIn, FP8, 1><<<rows, 256, 0, s>>>(y, scale, x, rows, K);
  } else if (K <= 2 * per_vec) {
    pertoken_quant_row_kernel<TIn, FP8, 2><<<rows, 256, 0, s>>>(y, scale, x, rows, K);
  } else if (K <= 4 * per_vec) {
    pertoken_quant_row_kernel<TIn, FP8, 4><<<rows, 256, 0, s>>>(y, scale, x, rows, K);
  } else if (K <= 8 * per_vec) {
    pertoken_quant_row_kernel<TIn, FP8, 8><<<rows, 256, 0, s>>>(y, scale, x, rows, K);
  } else {
    const int grid = rows < 148 * 16 ? rows : 148 * 16;
    pertoken_quant_kernel<TIn, FP8><<<grid, 256, 0, s>>>(y, scale, x, rows, K);
  }
}
template <typename TIn>
void launch_quant(uint8_t* y, float* scale, const TIn* x, int rows, int K, bool fp8, cudaStream_t s) {
  if (fp8) launch_quant_t<TIn, true>(y, scale, x, rows, K, s);
  else launch_quant_t<TIn, false>(y, scale, x, rows, K, s);
}

bool ranges_overlap(const void* a, const void* b, size_t bytes) {
  const uintptr_t x = reinterpret_cast<uintptr_t>(a), y = reinterpret_cast<uintptr_t>(b);
  return x < y + bytes && y < x + bytes;
}

// A wait on a barrier that nothing will ever complete, with a short limit: the
// same bounded wait the GEMM kernels use must give up, record ST_TIMEOUT in the
// status word and let the kernel return normally (no trap, no endless loop).
__global__ void selftest_wait_kernel(int* status, unsigned long long limit_ns) {
  __shared__ __align__(8) unsigned long long bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (!mbar_wait(smem_u32(&bar), 0, &abort_flag, nullptr, limit_ns)) atomicCAS(status, 0, ST_TIMEOUT);
  }
}

// ---------------------------------------------------------------------------
// Built-in scratch for callers that must not allocate device memory.
//
// The array lives in the library's device image: every GPU that loads the
// library carries these 8 MiB from load until the process exits, whether the
// entry point below is ever used or not.  On the host the symbol
// `g_static_scratch` is only a handle for the runtime, not an address a kernel
// can use; the usable device address is looked up once per device with
// cudaGetSymbolAddress and cached.
// ---------------------------------------------------------------------------
constexpr size_t STATIC_SCRATCH_BYTES = static_cast<size_t>(8) << 20;
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_SCRATCH_BYTES];

struct StaticScratchState {
  std::once_flag once;
  void* dev_ptr = nullptr;
  cudaError_t err = cudaSuccess;
};
StaticScratchState g_scratch_state[MAX_DEVICES];

// Device address of the scratch array on the current device (looked up on the
// first call per device, with that device current).
int static_scratch_address(void** out) {
  int dev = 0;
  CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= MAX_DEVICES) return FLYB200_E_UNSUPPORTED;
  StaticScratchState& st = g_scratch_state[dev];
  std::call_once(st.once, [&]() {
    void* p = nullptr;
    st.err = cudaGetSymbolAddress(&p, g_static_scratch);
    if (st.err == cudaSuccess) st.dev_ptr = p;
  });
  if (st.err != cudaSuccess) return cuda_fail(st.err, "cudaGetSymbolAddress(static scratch)");
  if (st.dev_ptr == nullptr) return FLYB200_E_CUDA;
  *out = st.dev_ptr;
  return FLYB200_OK;
}

}  // namespace

namespace flyb200 {
namespace host {
// Block-scaled GEMM (MXFP8, or MXFP4 with `fp4`) for up to 128 tokens on the small-M (weight-streaming)
// kernel; K = bytes of codes per row.
int gemm_mx_small(void* c, const void* a, const void* w, const void* sf_a, const void* sf_w, int M, int N, int K,
                  int outmode, bool fp4, void* stream) {
  DeviceState* st = nullptr;
  int rc = device_state(&st);
  if (rc) return rc;
  Plan plan;
  rc = make_plan(&plan, M, N, K, 1 << 8, 0, false, st->sms);
  if (rc) return rc;
  if (!plan.decode || plan.token_blocks != 1 || plan.w_rows != BLOCK_ROWS || plan.bn > 128) return FLYB200_E_UNSUPPORTED;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.w = static_cast<const uint8_t*>(w);
  p.c = c;
  p.M = M;
  p.N = N;
  p.K_bytes = K;
  p.epilogue = EPI_NONE;
  p.group_m = plan.group_m;
  p.split_k = plan.split_k;
  p.kb_per_split = plan.kb_per_split;
  p.reduce_mode = plan.reduce_mode;
  p.stages = plan.stages > 8 ? 8 : plan.stages;
  p.pdl = plan.pdl;
  p.prefetch = plan.prefetch;
  p.token_blocks = 1;
  p.sf_w = static_cast<const uint8_t*>(sf_w);
  p.sf_a = static_cast<const uint8_t*>(sf_a);
  p.sf_a_tiles = (M + 127) / 128;
  p.status = st->status;
  CUtensorMap tmA;
  rc = make_map(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a, static_cast<uint64_t>(K), static_cast<uint64_t>(M), KBLOCK_BYTES,
                plan.bn);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return host::launch_decode_kind(fp4 ? KIND_MXF4 : KIND_MXF8, outmode == OUT_FP16 ? OUT_FP16 : OUT_BF16, plan.bn, plan.w_rows, tmA,
                                  p, s);
}
int byte_matrix_map(CUtensorMap* m, const void* base, uint64_t row_bytes, uint64_t rows, uint32_t box_rows) {
  return make_map(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, base, row_bytes, rows, KBLOCK_BYTES, box_rows);
}
int status_word(int** out) {
  DeviceState* st = nullptr;
  const int rc = device_state(&st);
  if (rc) return rc;
  *out = st->status;
  return FLYB200_OK;
}
int record_cuda_error(cudaError_t e, const char* what) { return cuda_fail(e, what); }
int sm_count(int* out) {
  DeviceState* st = nullptr;
  const int rc = device_state(&st);
  if (rc) return rc;
  *out = st->sms;
  return FLYB200_OK;
}
}  // namespace host
}  // namespace flyb200

extern "C" {

int flyb200_gemm_a8w8(void* c, const void* a, const void* w_shuf, const float* scale_a, const float* scale_b,
                      const void* bias, int M, int N, int K, int in_dtype, int out_dtype, int epilogue,
                      int variant_hint, void* workspace, size_t workspace_bytes, void* stream) {
  if (out_dtype != FLYB200_OUT_BF16 && out_dtype != FLYB200_OUT_FP16) return FLYB200_E_BAD_ARG;
  const int eb = elem_bytes_of(in_dtype);
  if (eb == 1 && (!scale_a || !scale_b)) return FLYB200_E_BAD_ARG;
  if (eb == 2 && (scale_a || scale_b)) return FLYB200_E_BAD_ARG;
  return gemm_common(c, a, w_shuf, scale_a, scale_b, bias, M, N, K, in_dtype,
                     out_dtype == FLYB200_OUT_FP16 ? OUT_FP16 : OUT_BF16, epilogue, variant_hint, workspace,
                     workspace_bytes, stream);
}

int flyb200_gemm_a8w8_acc(void* acc, const void* a, const void* w_shuf, int M, int N, int K, int in_dtype,
                          int variant_hint, void* workspace, size_t workspace_bytes, void* stream) {
  if (in_dtype != FLYB200_DT_FP8 && in_dtype != FLYB200_DT_INT8) return FLYB200_E_UNSUPPORTED;
  return gemm_common(acc, a, w_shuf, nullptr, nullptr, nullptr, M, N, K, in_dtype, OUT_RAW32, FLYB200_EPI_NONE,
                     variant_hint, workspace, workspace_bytes, stream);
}

int flyb200_gemm_a8w8_static_scratch(void* c, const void* a, const void* w_shuf, const float* scale_a,
                                     const float* scale_b, const void* bias, int M, int N, int K, int in_dtype,
                                     int out_dtype, int epilogue, int split_k, void* stream) {
  if (out_dtype != FLYB200_OUT_BF16 && out_dtype != FLYB200_OUT_FP16) return FLYB200_E_BAD_ARG;
  if (in_dtype < FLYB200_DT_FP8 || in_dtype > FLYB200_DT_BF16 || split_k < 0 || split_k > 255) return FLYB200_E_BAD_ARG;
  const int eb = elem_bytes_of(in_dtype);
  if (eb == 1 && (!scale_a || !scale_b)) return FLYB200_E_BAD_ARG;
  if (eb == 2 && (scale_a || scale_b)) return FLYB200_E_BAD_ARG;
  if (M < 0 || N <= 0 || K <= 0) return FLYB200_E_BAD_ARG;
  if (M > 256) return FLYB200_E_UNSUPPORTED;  // only the small-M kernel has a split-K scratch
  if (!flyb200_layout_kind(N, K, eb)) return FLYB200_E_UNSUPPORTED;
  // every check that can fail comes before the first write to the shared array
  if (!c || !a || !w_shuf) return FLYB200_E_BAD_ARG;
  if (epilogue < FLYB200_EPI_NONE || epilogue > FLYB200_EPI_BIAS_GELU) return FLYB200_E_BAD_ARG;
  if (epilogue != FLYB200_EPI_NONE && !bias) return FLYB200_E_BAD_ARG;
  if (!aligned16(c) || !aligned16(a) || !aligned16(w_shuf)) return FLYB200_E_BAD_ALIGN;
  if (M == 0) return FLYB200_OK;

  const int bn = decode_bn_for(M);
  const int kb = (K * eb) / KBLOCK_BYTES;
  int split = split_k;
  if (split == 0) {
    // automatic: the usual factor, lowered until its partial sums fit the array
    DeviceState* st = nullptr;
    int rc = device_state(&st);
    if (rc) return rc;
    split = fill_sms_split_k(N, K * eb, st->sms);
    while (split > 1 && TICKET_BYTES + partial_bytes(split, N, bn) > STATIC_SCRATCH_BYTES) --split;
  }
  if (split > kb) split = kb;
  if (split < 1) split = 1;
  if (split > 1 && TICKET_BYTES + partial_bytes(split, N, bn) > STATIC_SCRATCH_BYTES) return FLYB200_E_SCRATCH_LIMIT;
  if ((N + BLOCK_ROWS - 1) / BLOCK_ROWS > static_cast<int>(TICKET_BYTES / sizeof(int))) return FLYB200_E_SCRATCH_LIMIT;

  void* scratch = nullptr;
  int rc = static_scratch_address(&scratch);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // The array still holds whatever the previous call left behind.  Only the
  // per-tile arrival counters have to start at zero (the partial sums are
  // fully overwritten before they are read), so those are cleared on the same
  // stream, ahead of the kernel.
  CUDA_TRY(cudaMemsetAsync(scratch, 0, TICKET_BYTES, s));
  // small-M kernel, reduction through the workspace, this split, no dependent launch
  // (and the tokens in one block, so that the size formula documented for this entry point holds)
  const int hint = (1 << 8) | (REDUCE_WORKSPACE << 12) | (2 << 28) | (1 << 30) | split;
  return gemm_common(c, a, w_shuf, scale_a, scale_b, bias, M, N, K, in_dtype,
                     out_dtype == FLYB200_OUT_FP16 ? OUT_FP16 : OUT_BF16, epilogue, hint, scratch, STATIC_SCRATCH_BYTES,
                     stream);
}

size_t flyb200_static_scratch_bytes(void) { return STATIC_SCRATCH_BYTES; }

int flyb200_gemm_a8w8_scatter(void* const* c_bufs, int n_bufs, int first_buf, long long c_pitch, long long c_col_offset,
                              const void* a, const void* w_shuf, const float* scale_a, const float* scale_b,
                              const void* bias, int M, int N, int K, int in_dtype, int out_dtype, int epilogue,
                              int variant_hint, void* stream) {
  if (!c_bufs || n_bufs < 1 || n_bufs > MAX_DESTINATIONS || first_buf < 0 || first_buf >= n_bufs) return FLYB200_E_BAD_ARG;
  if (out_dtype != FLYB200_OUT_BF16 && out_dtype != FLYB200_OUT_FP16) return FLYB200_E_BAD_ARG;
  if (in_dtype < FLYB200_DT_FP8 || in_dtype > FLYB200_DT_BF16) return FLYB200_E_BAD_ARG;
  if (epilogue < FLYB200_EPI_NONE || epilogue > FLYB200_EPI_BIAS_GELU) return FLYB200_E_BAD_ARG;
  if (epilogue != FLYB200_EPI_NONE && !bias) return FLYB200_E_BAD_ARG;
  const int eb = elem_bytes_of(in_dtype);
  if (eb == 1 && (!scale_a || !scale_b)) return FLYB200_E_BAD_ARG;
  if (eb == 2 && (scale_a || scale_b)) return FLYB200_E_BAD_ARG;
  if (!a || !w_shuf || M < 0 || N <= 0 || K <= 0) return FLYB200_E_BAD_ARG;
  if (c_col_offset < 0 || c_pitch < c_col_offset + N || (c_pitch % 8) != 0 || (c_col_offset % 8) != 0)
    return FLYB200_E_BAD_ARG;  // window inside the row, 16-byte aligned rows and window start
  if (!flyb200_layout_kind(N, K, eb)) return FLYB200_E_UNSUPPORTED;
  if (!aligned16(a) || !aligned16(w_shuf)) return FLYB200_E_BAD_ALIGN;
  for (int d = 0; d < n_bufs; ++d) {
    if (!c_bufs[d]) return FLYB200_E_BAD_ARG;
    if (!aligned16(c_bufs[d])) return FLYB200_E_BAD_ALIGN;
  }
  if (M == 0) return FLYB200_OK;

  DeviceState* st = nullptr;
  int rc = device_state(&st);
  if (rc) return rc;
  const int K_bytes = K * eb;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.w = static_cast<const uint8_t*>(w_shuf);
  p.sa = scale_a;
  p.sb = scale_b;
  p.bias = bias;
  p.c = c_bufs[0];
  p.M = M;
  p.N = N;
  p.K_bytes = K_bytes;
  p.epilogue = epilogue;
  p.group_m = hint_group(variant_hint) > 0 ? hint_group(variant_hint) : 32;
  p.split_k = 1;
  p.kb_per_split = K_bytes / KBLOCK_BYTES;
  p.bn = 256;
  p.rows_stages = host::rows_stages_for(256);
  p.n_dst = n_bufs;
  p.dst_first = first_buf;
  p.status = st->status;

  CUtensorMap tmA;
  rc = make_map(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a, static_cast<uint64_t>(K_bytes), static_cast<uint64_t>(M),
                KBLOCK_BYTES, BLOCK_ROWS);
  if (rc) return rc;
  OutputMaps outs;
  memset(&outs, 0, sizeof(outs));
  const CUtensorMapDataType odt =
      out_dtype == FLYB200_OUT_FP16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  for (int d = 0; d < n_bufs; ++d) {
    const uint8_t* base = static_cast<const uint8_t*>(c_bufs[d]) + static_cast<size_t>(c_col_offset) * 2;
    rc = make_window_map(&outs.m[d], odt, base, static_cast<uint64_t>(N), static_cast<uint64_t>(M),
                         static_cast<uint64_t>(c_pitch));
    if (rc) return rc;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return host::launch_rows_scatter_kind(kind_of(in_dtype), out_dtype == FLYB200_OUT_FP16 ? OUT_FP16 : OUT_BF16, tmA, outs, p,
                                        st->sms, s);
}

int flyb200_shuffle_weight(void* dst, const void* src, int N, int K, int elem_bytes, int src_layout, void* stream) {
  if (!dst || !src || N <= 0 || K <= 0) return FLYB200_E_BAD_ARG;
  if (!flyb200_layout_kind(N, K, elem_bytes)) return FLYB200_E_UNSUPPORTED;
  if (!aligned16(dst) || !aligned16(src)) return FLYB200_E_BAD_ALIGN;
  const size_t bytes = static_cast<size_t>(N) * K * elem_bytes;
  if (ranges_overlap(dst, src, bytes)) return FLYB200_E_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (src_layout == FLYB200_SRC_ROW_MAJOR) return launch_shuffle<FLYB200_SRC_ROW_MAJOR, false>(dst, src, N, K * elem_bytes, s);
  if (src_layout == FLYB200_SRC_MFMA_16x16) return launch_shuffle<FLYB200_SRC_MFMA_16x16, false>(dst, src, N, K * elem_bytes, s);
  return FLYB200_E_BAD_ARG;
}

int flyb200_unshuffle_weight(void* dst, const void* src, int N, int K, int elem_bytes, void* stream) {
  if (!dst || !src || N <= 0 || K <= 0) return FLYB200_E_BAD_ARG;
  if (!flyb200_layout_kind(N, K, elem_bytes)) return FLYB200_E_UNSUPPORTED;
  if (!aligned16(dst) || !aligned16(src)) return FLYB200_E_BAD_ALIGN;
  const size_t bytes = static_cast<size_t>(N) * K * elem_bytes;
  if (ranges_overlap(dst, src, bytes)) return FLYB200_E_BAD_ARG;
  return launch_shuffle<FLYB200_SRC_ROW_MAJOR, true>(dst, src, N, K * elem_bytes, static_cast<cudaStream_t>(stream));
}

int flyb200_pertoken_quant(void* y, float* scale, const void* x, int rows, int K, int x_dtype, int quant_dtype,
                           void* stream) {
  if (!y || !scale || !x || rows < 0 || K <= 0) return FLYB200_E_BAD_ARG;
  if (x_dtype < QX_F32 || x_dtype > QX_BF16) return FLYB200_E_BAD_ARG;
  if (quant_dtype != FLYB200_DT_FP8 && quant_dtype != FLYB200_DT_INT8) return FLYB200_E_BAD_ARG;
  const int vec = x_dtype == QX_F32 ? 4 : 8;
  if (K % vec != 0) return FLYB200_E_UNSUPPORTED;
  if (!aligned16(x) || (reinterpret_cast<uintptr_t>(y) & 7u) != 0) return FLYB200_E_BAD_ALIGN;
  if (rows == 0) return FLYB200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint8_t* yo = static_cast<uint8_t*>(y);
  const bool fp8 = quant_dtype == FLYB200_DT_FP8;
  if (x_dtype == QX_F32) {
    launch_quant<float>(yo, scale, static_cast<const float*>(x), rows, K, fp8, s);
  } else if (x_dtype == QX_F16) {
    launch_quant<__half>(yo, scale, static_cast<const __half*>(x), rows, K, fp8, s);
  } else {
    launch_quant<__nv_bfloat16>(yo, scale, static_cast<const __nv_bfloat16*>(x), rows, K, fp8, s);
  }
  CUDA_TRY(cudaGetLastError());
  return FLYB200_OK;
}

int flyb200_selftest_bounded_wait(unsigned int limit_us, void* stream) {
  if (limit_us == 0 || limit_us > 100000u) return FLYB200_E_BAD_ARG;  // at most 0.1 s
  DeviceState* st = nullptr;
  int rc = device_state(&st);
  if (rc) return rc;
  selftest_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(st->status,
                                                                      static_cast<unsigned long long>(limit_us) * 1000ull);
  CUDA_TRY(cudaGetLastError());
  return FLYB200_OK;
}

int flyb200_describe_plan(int M, int N, int K, int in_dtype, int variant_hint, int sm_count, int* out8) {
  if (!out8 || M <= 0 || N <= 0 || K <= 0 || sm_count <= 0) return FLYB200_E_BAD_ARG;
  if (in_dtype < FLYB200_DT_FP8 || in_dtype > FLYB200_DT_BF16) return FLYB200_E_BAD_ARG;
  const int eb = elem_bytes_of(in_dtype);
  if (!flyb200_layout_kind(N, K, eb)) return FLYB200_E_UNSUPPORTED;
  Plan plan;
  // planned as with an unlimited workspace: the answer says what would be needed
  int rc = make_plan(&plan, M, N, K * eb, variant_hint, static_cast<size_t>(-1) >> 1, true, sm_count);
  if (rc) return rc;
  out8[0] = plan.decode ? (plan.pair ? 5 : plan.w_rows == 64 ? 4 : 1) : (plan.two_sm ? 3 : plan.tall ? 6 : 2);
  out8[1] = plan.bn;
  out8[2] = plan.split_k;
  out8[3] = plan.kb_per_split;
  out8[4] = plan.reduce_mode;
  out8[5] = plan.decode ? plan.stages : (plan.two_sm ? ROWS2_STAGES : plan.tall ? host::ROWS_TALL_STAGES : host::rows_stages_for(plan.bn));
  out8[6] = plan.pdl;
  out8[7] = plan.token_blocks;
  return FLYB200_OK;
}

int flyb200_layout_kind(int N, int K, int elem_bytes) {
  if (elem_bytes != 1 && elem_bytes != 2) return 0;
  if (N <= 0 || K <= 0) return 0;
  if (N % 16 != 0) return 0;
  const long long kb = static_cast<long long>(K) * elem_bytes;
  if (kb % 128 != 0) return 0;
  if (kb > 0x7fffffffLL) return 0;
  return 1;
}

size_t flyb200_workspace_bytes(int M, int N, int K, int in_dtype, int variant_hint) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const int eb = elem_bytes_of(in_dtype);
  if (!flyb200_layout_kind(N, K, eb)) return 0;
  DeviceState* st = nullptr;
  if (device_state(&st)) return 0;
  // plan as the GEMM would with an unlimited workspace, then size for that plan
  Plan plan;
  if (make_plan(&plan, M, N, K * eb, variant_hint, static_cast<size_t>(-1) >> 1, true, st->sms)) return 0;
  if (!plan.decode || plan.reduce_mode != REDUCE_WORKSPACE) return 0;
  return TICKET_BYTES + partial_bytes(plan.split_k, N, plan.bn, plan.token_blocks);
}

int flyb200_read_status(int* out_status) {
  if (!out_status) return FLYB200_E_BAD_ARG;
  DeviceState* st = nullptr;
  int rc = device_state(&st);
  if (rc) return rc;
  CUDA_TRY(cudaDeviceSynchronize());
  int v = 0;
  CUDA_TRY(cudaMemcpy(&v, st->status, sizeof(int), cudaMemcpyDeviceToHost));
  if (v != 0) {
    int zero = 0;
    CUDA_TRY(cudaMemcpy(st->status, &zero, sizeof(int), cudaMemcpyHostToDevice));
  }
  *out_status = v;
  return FLYB200_OK;
}

const char* flyb200_strerror(int code) {
  switch (code) {
    case FLYB200_OK: return "ok";
    case FLYB200_E_BAD_ARG: return "bad argument";
    case FLYB200_E_BAD_ALIGN: return "pointer not 16-byte aligned";
    case FLYB200_E_CUDA: return "CUDA call failed";
    case FLYB200_E_TIMEOUT: return "bounded device-side wait expired";
    case FLYB200_E_UNSUPPORTED: return "unsupported shape or dtype (need N % 16 == 0 and K*elem_bytes % 128 == 0)";
    case FLYB200_E_SMEM_ALIGN: return "shared memory base not 1024-byte aligned";
    case FLYB200_E_WORKSPACE: return "workspace missing or too small for the requested split-K";
    case FLYB200_E_SCRATCH_LIMIT: return "problem needs more scratch than the library's built-in 8 MiB array holds";
  }
  return "unknown error";
}

const char* flyb200_last_cuda_error(void) { return g_cuda_err; }
int flyb200_version(void) { return 1; }

}  // extern "C"
