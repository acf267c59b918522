// C ABI of libmegaup.so: plans and launches for the two fused Ulysses exchange
// GEMMs, the cuMem-based symmetric arena, the slot hand-off flag barrier and
// the layout copies. Declarations and the reference seams they replace are in
// include/megaup.h.
//
// The driver API (cuMem*, cuTensorMapEncodeTiled) is reached through
// cudaGetDriverEntryPoint, so the library has no link-time dependency on
// libcuda and can be loaded (symbols inspected) on a machine without a GPU.

#include <cuda.h>
#include <cuda_runtime.h>
#include <unistd.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <algorithm>
#include <mutex>
#include <new>
#include <vector>

#include "../../include/megaup.h"
#include "mup_gemm.cuh"

namespace {

thread_local char g_last_error[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return code;
}

#define MUP_CUDA(expr)                                                                   \
  do {                                                                                   \
    cudaError_t e_ = (expr);                                                             \
    if (e_ != cudaSuccess)                                                               \
      return fail(MUP_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e_),  \
                  __FILE__, __LINE__);                                                   \
  } while (0)

// ---------------------------------------------------------------- driver API

struct DriverApi {
  decltype(&cuTensorMapEncodeTiled) tensor_map_encode_tiled = nullptr;
  decltype(&cuMemCreate) mem_create = nullptr;
  decltype(&cuMemRelease) mem_release = nullptr;
  decltype(&cuMemAddressReserve) mem_address_reserve = nullptr;
  decltype(&cuMemAddressFree) mem_address_free = nullptr;
  decltype(&cuMemMap) mem_map = nullptr;
  decltype(&cuMemUnmap) mem_unmap = nullptr;
  decltype(&cuMemSetAccess) mem_set_access = nullptr;
  decltype(&cuMemGetAllocationGranularity) mem_get_granularity = nullptr;
  decltype(&cuMemExportToShareableHandle) mem_export = nullptr;
  decltype(&cuMemImportFromShareableHandle) mem_import = nullptr;
  decltype(&cuGetErrorString) get_error_string = nullptr;
  bool ok = false;
  char error[256] = "";
};

template <typename Fn>
bool load_entry(const char* name, Fn* out, char* error, size_t error_len) {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult status;
  cudaError_t e = cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &status);
  if (e != cudaSuccess || status != cudaDriverEntryPointSuccess || fn == nullptr) {
    snprintf(error, error_len, "driver entry point %s unavailable (%s)", name,
             e != cudaSuccess ? cudaGetErrorString(e) : "not found");
    return false;
  }
  *out = reinterpret_cast<Fn>(fn);
  return true;
}

const DriverApi& driver() {
  static DriverApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    bool ok = true;
    char* err = api.error;
    const size_t n = sizeof(api.error);
    ok = ok && load_entry("cuTensorMapEncodeTiled", &api.tensor_map_encode_tiled, err, n);
    ok = ok && load_entry("cuMemCreate", &api.mem_create, err, n);
    ok = ok && load_entry("cuMemRelease", &api.mem_release, err, n);
    ok = ok && load_entry("cuMemAddressReserve", &api.mem_address_reserve, err, n);
    ok = ok && load_entry("cuMemAddressFree", &api.mem_address_free, err, n);
    ok = ok && load_entry("cuMemMap", &api.mem_map, err, n);
    ok = ok && load_entry("cuMemUnmap", &api.mem_unmap, err, n);
    ok = ok && load_entry("cuMemSetAccess", &api.mem_set_access, err, n);
    ok = ok && load_entry("cuMemGetAllocationGranularity", &api.mem_get_granularity, err, n);
    ok = ok && load_entry("cuMemExportToShareableHandle", &api.mem_export, err, n);
    ok = ok && load_entry("cuMemImportFromShareableHandle", &api.mem_import, err, n);
    ok = ok && load_entry("cuGetErrorString", &api.get_error_string, err, n);
    api.ok = ok;
  });
  return api;
}

int driver_fail(const char* what, CUresult r) {
  const char* msg = nullptr;
  if (driver().get_error_string != nullptr) driver().get_error_string(r, &msg);
  return fail(MUP_ERR_DRIVER, "%s failed: %s (CUresult %d)", what, msg ? msg : "?", static_cast<int>(r));
}

#define MUP_DRV(call, what)                     \
  do {                                          \
    CUresult r_ = (call);                       \
    if (r_ != CUDA_SUCCESS) return driver_fail(what, r_); \
  } while (0)

// BF16 row-major matrix [outer, inner] -> 2-D tiled tensor map with the
// 128-byte swizzle; box_inner is always 64 elements (128 bytes).
int encode_map(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer,
               uint64_t row_stride_elems, uint32_t box_inner, uint32_t box_outer) {
  const DriverApi& d = driver();
  if (!d.ok) return fail(MUP_ERR_DRIVER, "%s", d.error);
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0)
    return fail(MUP_ERR_BAD_ARG, "tensor base %p is not 16-byte aligned", base);
  if ((row_stride_elems * 2) % 16 != 0)
    return fail(MUP_ERR_BAD_ARG, "row stride of %llu BF16 is not a multiple of 16 bytes",
                static_cast<unsigned long long>(row_stride_elems));
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_elems * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t elem_strides[2] = {1, 1};
  CUresult r = d.tensor_map_encode_tiled(
      map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
      elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return driver_fail("cuTensorMapEncodeTiled", r);
  return MUP_OK;
}

// Rows per pull ticket: the largest power of two (at most 16) whose shard rows
// fit one batch of 512 sixteen-byte peer loads per warp.
int pull_rows_for(int shard) {
  if (const char* env = getenv("MEGA_UP_PULL_ROWS")) {
    const int forced = atoi(env);
    if ((forced == 1 || forced == 2 || forced == 4 || forced == 8 || forced == 16) &&
        forced * (shard / 8) <= mup::kPullMaxVecs)
      return forced;
  }
  const int vec_per_row = shard / 8;
  int rows = 16;
  while (rows > 1 && rows * vec_per_row > mup::kPullMaxVecs) rows /= 2;
  return rows;
}

// A shard row wider than one ticket is cut into equal column segments.
void set_pull_geometry(mup::GemmParams& p, int rows) {
  const int vec_per_row = p.shard / 8;
  p.pull_rows = pull_rows_for(p.shard);
  p.pull_segs = (vec_per_row + mup::kPullMaxVecs - 1) / mup::kPullMaxVecs;
  if (p.pull_segs < 1) p.pull_segs = 1;
  p.pull_seg_vecs = (vec_per_row + p.pull_segs - 1) / p.pull_segs;
  const int groups = (rows + p.pull_rows - 1) / p.pull_rows;
  p.total_tickets = groups * p.up * p.pull_segs;
  p.pull_up_shift = 0;
  while ((1 << p.pull_up_shift) < p.up) ++p.pull_up_shift;
  p.pull_pace_ns = 0;
  if (const char* env = getenv("MEGA_UP_PULL_PACE_NS")) p.pull_pace_ns = static_cast<unsigned int>(std::max(0, atoi(env)));
  if (p.pull_pace_ns > 100u) p.pull_pace_ns = 100u;  // at most 0.1 ms for the last warp of a grid
  p.pull_panel_shift = 0;
  while ((p.pull_rows << p.pull_panel_shift) < mup::kBlockM) ++p.pull_panel_shift;
}

int shape_rule(int64_t width, int up) {
  if (up != 2 && up != 4 && up != 8) return 1;
  if (width <= 0 || width % up) return 2;
  if (width % 256) return 3;
  if ((width / up) % 128) return 4;
  return 0;
}

int n_rotation(int rank, int up, int n_total, int tile_n) {
  const int n_tiles = (n_total + tile_n - 1) / tile_n;
  return ((rank * n_tiles + up - 1) / up) % n_tiles;
}

// Translate the C-ABI hand-off description; `participants` = arrivals this launch adds to the counter.
int fill_sync(mup::SyncParams* sp, mup_sync* sync, unsigned long long participants) {
  memset(sp, 0, sizeof(*sp));
  if (sync == nullptr) return MUP_OK;
  if (sync->peer_flags == nullptr || sync->up < 1 || sync->up > mup::kMaxPeers || sync->rank < 0 ||
      sync->rank >= sync->up)
    return fail(MUP_ERR_BAD_ARG, "bad hand-off description (flags, up or rank)");
  if (sync->signal_epoch != 0 && sync->done_counter == nullptr)
    return fail(MUP_ERR_BAD_ARG, "a hand-off that signals needs a done counter");
  if (reinterpret_cast<uintptr_t>(sync->done_counter) % 8)
    return fail(MUP_ERR_BAD_ARG, "done counter must be 8-byte aligned");
  for (int i = 0; i < sync->up; ++i) {
    if (sync->peer_flags[i] == nullptr) return fail(MUP_ERR_BAD_ARG, "flag array %d is null", i);
    sp->flags[i] = static_cast<uint32_t*>(sync->peer_flags[i]);
  }
  sp->done = static_cast<unsigned long long*>(sync->done_counter);
  sp->done_target = sync->done_before + participants;
  sp->status = static_cast<uint32_t*>(sync->status_device_ptr);
  sp->timeout_ns = sync->timeout_ns;
  sp->wait_epoch = sync->wait_epoch;
  sp->signal_epoch = sync->signal_epoch;
  sp->up = sync->up;
  sp->rank = sync->rank;
  sync->done_after = (sync->signal_epoch != 0) ? sp->done_target : sync->done_before;
  return MUP_OK;
}

// Upper bound on the CTAs of plans created by this thread from now on (0: none).
thread_local int g_max_ctas_option = 0;

struct DeviceInfo {
  int sms = 0;
  int cc_major = 0;
};

int query_device(int device, DeviceInfo* info) {
  MUP_CUDA(cudaDeviceGetAttribute(&info->sms, cudaDevAttrMultiProcessorCount, device));
  MUP_CUDA(cudaDeviceGetAttribute(&info->cc_major, cudaDevAttrComputeCapabilityMajor, device));
  return MUP_OK;
}

template <int G, int MODE>
int configure_kernel(int* max_clusters) {
  auto kernel = mup::fused_exchange_gemm_kernel<G, MODE, true>;
  const int smem = mup::GemmCfg<G>::kSmemBytes;
  MUP_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  MUP_CUDA(cudaFuncSetAttribute(mup::fused_exchange_gemm_kernel<G, MODE, false>,
                                cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  if (G == 2) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(2, 1, 1);
    cfg.blockDim = dim3(mup::kernel_threads(MODE), 1, 1);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    MUP_CUDA(cudaOccupancyMaxActiveClusters(&n, kernel, &cfg));
    *max_clusters = n;
  }
  return MUP_OK;
}

// Programmatic dependent launch: every kernel of this library is launched with
// the programmatic-serialization attribute, lets its successor be scheduled at
// once (griddepcontrol.launch_dependents at entry) and waits for its
// predecessor with griddepcontrol.wait before it touches global memory, so the
// launch latency and the set-up of a kernel (barrier init, TMEM allocation,
// cluster sync) hide behind the tail of the kernel before. A kernel launched
// by someone else after these waits for their full completion as usual.
// Measured on 2 B200s: peer-write call 171.8 -> 170.5 us, pull call 190.4 ->
// 187.9 us, both back to back 367.3 -> 365.3 us. MEGA_UP_PDL=0 turns it off.
bool pdl_enabled() {
  static int cached = -1;
  if (cached < 0) {
    const char* env = getenv("MEGA_UP_PDL");
    cached = (env != nullptr && atoi(env) == 0) ? 0 : 1;
  }
  return cached == 1;
}

template <int G, int MODE>
int launch_kernel(const mup::GemmParams& params, int grid, cudaStream_t stream) {
  // lists without two-accumulator items run the instantiation without their code
  auto kernel = params.max_item_cols > mup::kBlockN ? mup::fused_exchange_gemm_kernel<G, MODE, true>
                                                    : mup::fused_exchange_gemm_kernel<G, MODE, false>;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(mup::kernel_threads(MODE), 1, 1);
  cfg.dynamicSmemBytes = mup::GemmCfg<G>::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  int n = 0;
  if (G == 2) {
    attrs[n].id = cudaLaunchAttributeClusterDimension;
    attrs[n].val.clusterDim.x = G;
    attrs[n].val.clusterDim.y = 1;
    attrs[n].val.clusterDim.z = 1;
    ++n;
  }
  if (pdl_enabled()) {
    attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = n;
  MUP_CUDA(cudaLaunchKernelEx(&cfg, kernel, params));
  return MUP_OK;
}

// Launch of the small kernels (barrier, layout copies), with the same attribute.
template <typename... KArgs, typename... Args>
cudaError_t launch_small(void (*kernel)(KArgs...), int grid, int block, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(block, 1, 1);
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Shared plan state of the two operators.
struct PlanCore {
  mup::GemmParams params;
  int device = 0;
  int cta_group = 1;
  int grid = 0;
  int smem_bytes = 0;
  std::vector<uint32_t> host_items;  // the work-item list (host copy)
  void* device_items = nullptr;      // the same list in device memory (owned)
  double model_cycles = 0;           // critical path the time model predicts
  ~PlanCore() {
    if (device_items != nullptr) cudaFree(device_items);
  }
};

int check_common(int device, int rows, int n, int k, int up, int rank, const void* weight,
                 const void* bias, int cta_group) {
  if (rows <= 0 || n <= 0 || k <= 0) return fail(MUP_ERR_BAD_ARG, "rows, n and k must be positive");
  if (up != 2 && up != 4 && up != 8) return fail(MUP_ERR_BAD_ARG, "up must be 2, 4 or 8, got %d", up);
  if (rank < 0 || rank >= up) return fail(MUP_ERR_BAD_ARG, "rank %d outside [0, %d)", rank, up);
  if (n % 256) return fail(MUP_ERR_BAD_ARG, "n=%d must be a multiple of 256", n);
  if (k % 8) return fail(MUP_ERR_BAD_ARG, "k=%d must be a multiple of 8", k);
  if (weight == nullptr) return fail(MUP_ERR_BAD_ARG, "weight is null");
  if (bias != nullptr && reinterpret_cast<uintptr_t>(bias) % 16)
    return fail(MUP_ERR_BAD_ARG, "bias must be 16-byte aligned");
  if (cta_group < 0 || cta_group > 2) return fail(MUP_ERR_BAD_ARG, "cta_group must be 0, 1 or 2");
  DeviceInfo info;
  int rc = query_device(device, &info);
  if (rc != MUP_OK) return rc;
  if (info.cc_major != 10)
    return fail(MUP_ERR_UNSUPPORTED, "device %d has compute capability %d.x; sm_100 is required",
                device, info.cc_major);
  return MUP_OK;
}

// ---------------------------------------------------------------- schedule
//
// The output is cut into work items of 128*G rows by 64..512 columns; CTA
// (pair) c runs items c, c + slots, ... of the list built here (or, for long
// lists, draws them in list order: item_feed_enabled). Candidate lists
// are rated with a time model calibrated on B200 (SM cycles at 1.6-1.7 GHz,
// 4096 x 5120 x 5120, CTA pairs). One K step of an item of `cols` columns costs
//
//   max(2 * cols, (3000 + 2 * cols) / stages)
//
// : the tensor pipe needs 2 * cols cycles, and a stage is refilled only about
// 3000 cycles after the MMAs released it (1.8 us: every K step touches lines no
// SM has read in this round, so a stage completes at DRAM latency), which the
// stages in flight cover only partly (measured per K step: 128-wide 410 with 8
// stages, 192-wide 530 with 7, 256-wide 565-585 with 6). An item costs 1200
// cycles on top (pipeline fill, accumulator hand-over); an item of two
// accumulators (wider than 256 columns) 15000, because all of TMEM belongs to
// it and the K loop of the next item cannot start before the epilogue has read
// an accumulator (with that figure the model reproduces what was measured: two
// accumulators lose at K = 4096 and 5120 and win at K = 8192, where the
// 16384 x 8192 x 8192 pull runs 10 % faster with 512-wide items); a change of
// stage geometry between two items of a CTA costs another 3000.
// Candidates: every M tile cut into q equal items, for a range of q; lists of
// r * slots items for a few r, where the M tiles differ by at most one item; and
// each of those with the items of a partly filled last round cut into f pieces
// (f * leftover <= slots), which keeps more SMs busy at the end. The candidate
// with the shortest critical path under round-robin assignment wins. Inside
// every round after the first the items are then dealt so that the CTA (pair)
// with the most work so far receives the cheapest item (`kNoItem` entries mark
// the pairs that sit out a partly filled last round). A peer-write list of four
// rounds or more may instead be re-ordered into bands of M tiles (maybe_band in
// choose_schedule).
// Measured and rejected: asking L2 for the boxes of later K steps with
// cp.async.bulk.prefetch.tensor from the TMA producer, 4 to 24 K steps ahead,
// by every CTA or by one CTA per line: the kernel went from 151 to 196-207 us
// (the MMA warp then waits for operands 3.5 times as long).
// Tuning overrides (environment): MEGA_UP_ITEM_UNITS=u forces items of u*64
// columns, MEGA_UP_ROUNDS=r forces the number of rounds, MEGA_UP_SPLIT_TAIL=0
// keeps the last round whole, MEGA_UP_BALANCE=0 keeps list order, MEGA_UP_BAND=b
// forces bands of b M tiles (peer-write only; 1 = row by row),
// MEGA_UP_BAND_INTERLEAVE=0 keeps a band's columns in order, MEGA_UP_ITEM_FEED=0/1
// forces the fixed assignment / the item feed.

int env_int(const char* name, int fallback) {
  const char* env = getenv(name);
  return (env != nullptr && *env) ? atoi(env) : fallback;
}

// Whether the CTAs (pairs) draw their items from the list as they become free
// (GemmParams::feed; the list then stays in natural order) or CTA c runs items
// c, c + grid, ... of a list dealt by balance_rounds. Drawing pays for lists of
// many rounds (65536 x 5120 x 5120: 2244 against 2270 us; 8192 x 6144 x 4096
// pull: 296.9 against 299.4 us), where the SMs drift apart; on 4096 x 5120 x
// 5120 it changes nothing (the slowest CTA pair is the one with a fifth, narrow
// item either way) and on one-round lists the first draw sits on the critical
// path (18 -> 25 us). MEGA_UP_ITEM_FEED=0/1 forces it off/on.
constexpr size_t kFeedMinRounds = 16;
bool item_feed_enabled(size_t items, int slots) {
  const int forced = env_int("MEGA_UP_ITEM_FEED", -1);
  if (forced >= 0) return forced != 0;
  return items >= kFeedMinRounds * static_cast<size_t>(slots);
}

struct Schedule {
  std::vector<uint32_t> items;
  bool fed = false;  // the CTAs draw the items (natural order) instead of a fixed assignment
  int max_cols = 0;
  double critical_cycles = 0;
};

// Load latency the stages in flight have to cover, in SM cycles (about 1.8 us:
// every K step touches lines no SM has read in this round of items).
constexpr double kModelLoadLatency = 3000.0;

// What the time model needs to know beside an item's width.
struct ModelShape {
  int k_tiles = 1;
  int g = 2;
  double latency = kModelLoadLatency;
  bool narrow_class = true;  // items of at most 128 columns get the 8-stage geometry
};

double item_cycles(int units, const ModelShape& shape) {
  const int cols = units * mup::kUnit;
  const double tensor = 2.0 * cols;
  const int stages = mup::tile_stages(mup::stage_class_cols(cols, shape.narrow_class), shape.g);
  const double step = std::max(tensor, (shape.latency + tensor) / stages);
  const double fixed = cols > mup::kBlockN ? 15000.0 : 1200.0;
  return shape.k_tiles * step + fixed;
}

int item_stage_class(uint32_t e) {
  // lists that change geometry have wide items; their narrow items use the 256-column one
  return mup::stage_class_cols((static_cast<int>((e >> 26) & 0x7u) + 1) * mup::kUnit, false);
}

// The 128-column stage geometry (8 stages) is used only by lists made of such
// items alone; see kFlagNoNarrowClass.
bool list_uses_narrow_class(const std::vector<uint32_t>& items) {
  for (uint32_t e : items)
    if (e != mup::kNoItem && ((e >> 26) & 0x7u) + 1u > 2u) return false;
  return true;
}

// Items of one M tile: `q` items covering `units` 64-column units, the first
// units % q of them one unit wider; emitted from position `start` cyclically.
void emit_row(std::vector<uint32_t>* out, int m_idx, int units, int q, int start) {
  const int base = units / q, extra = units % q;
  for (int j = 0; j < q; ++j) {
    const int pos = (start + j) % q;
    const int n0 = pos * base + std::min(pos, extra);
    const int w = base + (pos < extra ? 1 : 0);
    out->push_back(mup::encode_item(m_idx, n0, w));
  }
}

double list_item_cycles(uint32_t e, const ModelShape& shape) {
  if (e == mup::kNoItem) return 0.0;
  return item_cycles(static_cast<int>((e >> 26) & 0x7u) + 1, shape);
}

// `start_cycles_per_m_tile` (pull mode): a CTA pair cannot start before the rows
// of its first item have arrived, and rows arrive in ascending order. Lists of
// wide items spread their first round over twice as many rows: on two and four
// GPUs the first panel gate then opened after 32-47 us on average instead of
// 23-26 us and the pull call of 4096 x 5120 x 5120 took 3-8 us longer, although
// with peers emulated on one GPU (rows arrive at HBM speed) the wide list was
// 5 us faster.
double critical_path(const std::vector<uint32_t>& items, int slots, ModelShape shape,
                     double start_cycles_per_m_tile) {
  std::vector<double> load(static_cast<size_t>(slots), 0.0);
  if (start_cycles_per_m_tile > 0.0) {
    for (size_t c = 0; c < static_cast<size_t>(slots) && c < items.size(); ++c)
      if (items[c] != mup::kNoItem) load[c] = start_cycles_per_m_tile * ((items[c] & 0x3FFFu) + 1u);
  }
  std::vector<int> last_class(static_cast<size_t>(slots), 0);
  shape.narrow_class = list_uses_narrow_class(items);
  for (size_t i = 0; i < items.size(); ++i) {
    if (items[i] == mup::kNoItem) continue;
    const size_t c = i % static_cast<size_t>(slots);
    load[c] += list_item_cycles(items[i], shape);
    // a change of stage geometry between two items drains the pipeline once
    const int cls = item_stage_class(items[i]);
    if (last_class[c] != 0 && last_class[c] != cls) load[c] += shape.latency;
    last_class[c] = cls;
  }
  return *std::max_element(load.begin(), load.end());
}

// Deal the items of every round after the first so that the slot with the most
// work so far gets the cheapest item of the round; a partly filled last round
// goes to the least loaded slots and the others get kNoItem. The first round
// keeps list order (in pull mode its items are the first panels to arrive).
void balance_rounds(std::vector<uint32_t>* items, int slots, ModelShape shape, double start_cycles_per_m_tile) {
  const size_t n = items->size();
  if (n <= static_cast<size_t>(slots)) return;
  shape.narrow_class = list_uses_narrow_class(*items);
  std::vector<double> load(static_cast<size_t>(slots), 0.0);
  // Pull mode: a CTA pair cannot start before the rows of its first item have
  // arrived, and rows arrive in ascending order at the rate the peers deliver
  // them, so the pairs that start on later rows begin with that much "work".
  if (start_cycles_per_m_tile > 0.0) {
    for (int c = 0; c < slots; ++c) {
      const uint32_t e = (*items)[static_cast<size_t>(c)];
      if (e != mup::kNoItem) load[static_cast<size_t>(c)] = start_cycles_per_m_tile * ((e & 0x3FFFu) + 1u);
    }
  }
  std::vector<uint32_t> out;
  out.reserve((n + slots - 1) / slots * slots);
  for (size_t r0 = 0; r0 < n; r0 += slots) {
    const size_t count = std::min(n - r0, static_cast<size_t>(slots));
    std::vector<uint32_t> round(items->begin() + r0, items->begin() + r0 + count);
    std::vector<uint32_t> placed(static_cast<size_t>(slots), mup::kNoItem);
    if (r0 == 0) {
      for (size_t i = 0; i < count; ++i) placed[i] = round[i];
    } else {
      std::vector<int> order(static_cast<size_t>(slots));
      for (int c = 0; c < slots; ++c) order[static_cast<size_t>(c)] = c;
      // most loaded slot first; ties keep the slot order
      std::stable_sort(order.begin(), order.end(),
                       [&](int a, int b) { return load[static_cast<size_t>(a)] > load[static_cast<size_t>(b)]; });
      // cheapest item first; ties keep list order
      std::stable_sort(round.begin(), round.end(), [&](uint32_t a, uint32_t b) {
        return list_item_cycles(a, shape) < list_item_cycles(b, shape);
      });
      // with fewer items than slots the most loaded slots sit the round out
      const size_t skip = static_cast<size_t>(slots) - count;
      for (size_t i = 0; i < count; ++i) placed[static_cast<size_t>(order[skip + i])] = round[i];
    }
    for (int c = 0; c < slots; ++c) {
      load[static_cast<size_t>(c)] += list_item_cycles(placed[static_cast<size_t>(c)], shape);
      out.push_back(placed[static_cast<size_t>(c)]);
    }
  }
  while (!out.empty() && out.back() == mup::kNoItem) out.pop_back();
  items->swap(out);
}

struct ListOptions {
  int units = 0;  // 64-column units per M tile
  int up = 1, rank = 0;
  bool rotate = false;  // peer-write: each rank starts every M tile at its own column block
  int band = 1;
  int slots = 1;
  ModelShape shape;
  double start_cycles_per_m_tile = 0.0;
};

// Cut every item of a partly filled last round into `pieces` narrower items (as
// equal as 64-column units allow), so that the round keeps more SMs busy.
void split_last_round(std::vector<uint32_t>* items, int slots, int pieces) {
  const size_t leftover = items->size() % static_cast<size_t>(slots);
  if (pieces < 2 || leftover == 0 || leftover * pieces > static_cast<size_t>(slots)) return;
  std::vector<uint32_t> tail(items->end() - static_cast<long>(leftover), items->end());
  items->resize(items->size() - leftover);
  for (uint32_t e : tail) {
    const int m = static_cast<int>(e & 0x3FFFu), n0 = static_cast<int>((e >> 14) & 0xFFFu);
    const int w = static_cast<int>((e >> 26) & 0x7u) + 1;
    const int f = std::min(pieces, w);
    int at = n0;
    for (int j = 0; j < f; ++j) {
      const int piece = w / f + (j < w % f ? 1 : 0);
      items->push_back(mup::encode_item(m, at, piece));
      at += piece;
    }
  }
}

// q_of_row[m] items for M tile m; the last round's items cut into `tail_pieces`.
Schedule build_list(const std::vector<int>& q_of_row, const ListOptions& o, int tail_pieces) {
  Schedule s;
  const int m_tiles = static_cast<int>(q_of_row.size());
  std::vector<std::vector<uint32_t>> rows(static_cast<size_t>(m_tiles));
  for (int m = 0; m < m_tiles; ++m) {
    const int q = q_of_row[m];
    const int start = o.rotate ? ((o.rank * q + o.up - 1) / o.up) % q : 0;
    emit_row(&rows[m], m, o.units, q, start);
  }
  if (o.band > 1 && o.rotate && o.up > 1 && env_int("MEGA_UP_BAND_INTERLEAVE", 1) != 0) {
    // A band walks its columns one after the other, so without this step it would
    // store to one destination rank for a long stretch (NVLink then sees the
    // exchange in bursts). Reorder every row so that consecutive items go to
    // different destinations: the 1st item of every destination's column block
    // (in rotation order), then the 2nd of each, ...
    const int shard_units = o.units / o.up;
    for (int m = 0; m < m_tiles; ++m) {
      std::vector<uint32_t>& row = rows[m];
      std::vector<int> seen(static_cast<size_t>(o.up), 0);
      std::vector<std::pair<int, size_t>> key(row.size());
      for (size_t j = 0; j < row.size(); ++j) {
        const int dest = std::min(o.up - 1, static_cast<int>((row[j] >> 14) & 0xFFFu) / shard_units);
        key[j] = {seen[static_cast<size_t>(dest)]++, j};
      }
      std::stable_sort(key.begin(), key.end(),
                       [](const std::pair<int, size_t>& x, const std::pair<int, size_t>& y) { return x.first < y.first; });
      std::vector<uint32_t> reordered(row.size());
      for (size_t j = 0; j < row.size(); ++j) reordered[j] = row[key[j].second];
      row.swap(reordered);
    }
  }
  if (o.band <= 1) {
    for (int m = 0; m < m_tiles; ++m) s.items.insert(s.items.end(), rows[m].begin(), rows[m].end());
  } else {
    for (int m0 = 0; m0 < m_tiles; m0 += o.band) {
      const int m1 = std::min(m_tiles, m0 + o.band);
      size_t longest = 0;
      for (int m = m0; m < m1; ++m) longest = std::max(longest, rows[m].size());
      // every other band walks its columns backwards (a serpentine): consecutive
      // bands then share W boxes at the turn
      const bool backwards = ((m0 / o.band) & 1) != 0;
      for (size_t jj = 0; jj < longest; ++jj) {
        const size_t j = backwards ? longest - 1 - jj : jj;
        for (int m = m0; m < m1; ++m)
          if (j < rows[m].size()) s.items.push_back(rows[m][j]);
      }
    }
  }
  split_last_round(&s.items, o.slots, tail_pieces);
  s.max_cols = 0;
  for (uint32_t e : s.items) s.max_cols = std::max(s.max_cols, (static_cast<int>((e >> 26) & 0x7u) + 1) * mup::kUnit);
  s.fed = item_feed_enabled(s.items.size(), o.slots);
  if (env_int("MEGA_UP_BALANCE", 1) != 0 && !s.fed && o.band <= 1)
    balance_rounds(&s.items, o.slots, o.shape, o.start_cycles_per_m_tile);
  s.critical_cycles = critical_path(s.items, o.slots, o.shape, o.start_cycles_per_m_tile);
  return s;
}

Schedule choose_schedule(int mode, int m_tiles, int n, int k_tiles, int up, int rank, int g, int slots) {
  ListOptions o;
  o.units = n / mup::kUnit;
  o.up = up;
  o.rank = rank;
  o.rotate = (mode == mup::MODE_PEER_WRITE);
  // A peer-write list walks bands of 8 M tiles column by column, every other
  // band backwards, with consecutive items of a row going to different
  // destination ranks (MEGA_UP_BAND=b changes the band, 1 = row by row). The
  // CTA pairs of a round then work on a squarer patch of the output (8 row tiles
  // x 9 column tiles instead of 3.7 x 20), more operand loads hit L2 (ncu: DRAM
  // reads 138 MB for such a raster against 190 MB row by row) and a stage comes
  // back sooner. 4096 x 5120 x 5120, kernel alone: 143.4 against 147.3 us with
  // emulated peers (cuBLAS 143.6), 150.3 against 152.7 us on two GPUs, 153.9
  // against 155.7 us on four. Without the alternation of destinations a band
  // stores to one rank for a long stretch and NVLink sees the exchange in
  // bursts: 154.3 us and a call 3-5 us slower on two GPUs. Banded lists are
  // not dealt by balance_rounds (143.4 against 144.7-145.4 us).
  o.band = o.rotate ? std::max(1, env_int("MEGA_UP_BAND", 8)) : 1;
  o.slots = slots;
  o.shape.k_tiles = k_tiles;
  o.shape.g = g;
  o.shape.latency = kModelLoadLatency;
  if (const char* env = getenv("MEGA_UP_MODEL_LATENCY")) o.shape.latency = atof(env);
  const int units = o.units;
  const int max_units = mup::max_item_cols(g) / mup::kUnit;
  const int q_min = (units + max_units - 1) / max_units;
  // Pull mode: SM cycles until one more M tile of rows has been pulled. The
  // remote share of a tile's bytes at the rate peer loads deliver over NVLink
  // (about 600 GB/s of the 770 GB/s a peer copy measures = 380 bytes per SM
  // cycle at 1.6 GHz; MEGA_UP_PULL_BPC overrides, 0 ignores the start-up skew).
  if (mode == mup::MODE_PULL && up > 1) {
    double pull_bpc = 380.0;
    if (const char* env = getenv("MEGA_UP_PULL_BPC")) pull_bpc = atof(env);
    if (pull_bpc > 0.0)
      o.start_cycles_per_m_tile =
          static_cast<double>(mup::kBlockM) * g * k_tiles * mup::kBlockK * 2.0 * (up - 1) / up / pull_bpc;
  }
  const bool may_split = env_int("MEGA_UP_SPLIT_TAIL", 1) != 0;
  // The list is chosen among row-by-row candidates; a peer-write list may then
  // be re-ordered into bands (below).
  ListOptions banded = o;
  o.band = 1;
  Schedule best;
  std::vector<int> best_q;
  int best_pieces = 1;
  bool have = false;
  // a list as it is, and with its last round cut into 2, 3 and 4 pieces per item
  auto consider = [&](const std::vector<int>& q_of_row, int pieces) {
    Schedule cand = build_list(q_of_row, o, pieces);
    if (!have || cand.critical_cycles < best.critical_cycles * 0.999 ||
        (cand.critical_cycles <= best.critical_cycles * 1.001 && cand.items.size() < best.items.size())) {
      best = std::move(cand);
      best_q = q_of_row;
      best_pieces = pieces;
      have = true;
    }
  };
  auto consider_with_tails = [&](const std::vector<int>& q_of_row) {
    consider(q_of_row, 1);
    long long total = 0;
    for (int q : q_of_row) total += q;
    const long long leftover = total % slots;
    if (!may_split || leftover == 0) return;
    for (int pieces = 2; pieces <= 4 && leftover * pieces <= slots; ++pieces) consider(q_of_row, pieces);
  };
  // Banding pays when the CTA pairs of a round then work on a clearly smaller
  // set of operand rows (A rows + W rows in flight; the threshold of 1.3 sits
  // between the shapes where it measured faster and slower):
  //   4096 x 5120 x 5120    row by row 144.8 us, banded 142.2   (ratio 1.37)
  //   8192 x 6144 x 4096               265.4            263.5   (1.57)
  //   16384 x 8192 x 8192              1440             1405    (1.38)
  //   65536 x 5120 x 5120              2181             2150    (1.37)
  //   8192 x 4096 x 4096               168.9            171.6   (1.19)
  // and only for lists of four rounds or more: with two rounds the even deal
  // of balance_rounds matters more (2048 x 5120 x 5120: 76.3 us dealt, 82.7 banded).
  auto maybe_band = [&]() {
    if (!have || banded.band <= 1 || best.items.size() < 4 * static_cast<size_t>(slots)) return;
    const bool forced = getenv("MEGA_UP_BAND") != nullptr;
    const double q = static_cast<double>(best.items.size()) / m_tiles;  // items per row tile
    const double item_cols = static_cast<double>(n) / q;
    const double tile_rows = static_cast<double>(mup::kBlockM) * g;
    const double rows_wide = std::max(1.0, slots / q) * tile_rows + std::min(q, static_cast<double>(slots)) * item_cols;
    const double band_rows = std::min(banded.band, m_tiles);
    const double band_wide = band_rows * tile_rows + std::min(q, slots / band_rows) * item_cols;
    if (forced || rows_wide >= 1.3 * band_wide) best = build_list(best_q, banded, best_pieces);
  };
  auto uniform = [&](int q) { return std::vector<int>(static_cast<size_t>(m_tiles), q); };
  const int forced_units = env_int("MEGA_UP_ITEM_UNITS", 0);
  if (forced_units >= 1 && forced_units <= max_units) {
    consider_with_tails(uniform(std::min(units, (units + forced_units - 1) / forced_units)));
    maybe_band();
    return best;
  }
  const int forced_rounds = env_int("MEGA_UP_ROUNDS", 0);
  if (forced_rounds <= 0) {
    const int q_hi = std::min(units, q_min + 24);
    for (int q = q_min; q <= q_hi; ++q) consider_with_tails(uniform(q));
  }
  const long long min_items = static_cast<long long>(m_tiles) * q_min;
  const int r_lo = forced_rounds > 0 ? forced_rounds : static_cast<int>((min_items + slots - 1) / slots);
  const int r_hi = forced_rounds > 0 ? forced_rounds : r_lo + 3;
  for (int r = std::max(1, r_lo); r <= r_hi; ++r) {
    const long long target = static_cast<long long>(r) * slots;
    long long q_lo = target / m_tiles;
    long long rows_hi = target - q_lo * m_tiles;  // this many M tiles get one item more
    if (q_lo < q_min) {
      q_lo = q_min;
      rows_hi = 0;
    }
    if (q_lo >= units) {
      q_lo = units;
      rows_hi = 0;
    }
    std::vector<int> q_of_row(static_cast<size_t>(m_tiles), static_cast<int>(q_lo));
    for (long long m = 0; m < rows_hi; ++m) q_of_row[static_cast<size_t>(m)] = static_cast<int>(q_lo + 1);
    consider_with_tails(q_of_row);
    if (q_lo >= units) break;
  }
  maybe_band();
  return best;
}

// Fill the geometry shared by both modes, build the schedule and size the grid.
template <int MODE>
int finish_core(PlanCore* core, int device, int rows, int n, int k, int up, int rank,
                int cta_group) {
  DeviceInfo info;
  int rc = query_device(device, &info);
  if (rc != MUP_OK) return rc;
  const int g = (cta_group == 0) ? 2 : cta_group;  // the CTA pair halves W traffic per SM
  mup::GemmParams& p = core->params;
  p.M = rows;
  p.N = n;
  p.K = k;
  p.up = up;
  p.rank = rank;
  p.k_tiles = (k + mup::kBlockK - 1) / mup::kBlockK;
  const int m_tiles = (rows + mup::kBlockM * g - 1) / (mup::kBlockM * g);
  if (m_tiles > mup::kMaxItemMTiles || n / mup::kUnit > mup::kMaxItemNUnits)
    return fail(MUP_ERR_UNSUPPORTED, "rows=%d or n=%d exceeds the schedule's range (%d row tiles, %d columns)", rows,
                n, mup::kMaxItemMTiles, mup::kMaxItemNUnits * mup::kUnit);
  int max_clusters = 0;
  int slots = info.sms;
  if (g == 1) {
    rc = configure_kernel<1, MODE>(&max_clusters);
    if (rc != MUP_OK) return rc;
    core->smem_bytes = mup::GemmCfg<1>::kSmemBytes;
  } else {
    rc = configure_kernel<2, MODE>(&max_clusters);
    if (rc != MUP_OK) return rc;
    if (max_clusters <= 0) return fail(MUP_ERR_UNSUPPORTED, "no 2-CTA cluster fits on device %d", device);
    slots = std::min(info.sms / 2, max_clusters);
    core->smem_bytes = mup::GemmCfg<2>::kSmemBytes;
  }
  // A caller that shares the GPU with other kernels can leave SMs free: a grid
  // that is not resident at once would stall at its first panel gates until
  // the missing CTAs' pull warps get an SM.
  if (g_max_ctas_option > 0) slots = std::max(1, std::min(slots, g_max_ctas_option / g));
  Schedule schedule = choose_schedule(MODE, m_tiles, n, p.k_tiles, up, rank, g, slots);
  const int clusters = static_cast<int>(std::min<size_t>(static_cast<size_t>(slots), schedule.items.size()));
  core->grid = clusters * g;
  core->device = device;
  core->cta_group = g;
  core->host_items = std::move(schedule.items);
  core->model_cycles = schedule.critical_cycles;
  p.num_items = static_cast<int>(core->host_items.size());
  p.max_item_cols = schedule.max_cols;
  p.row_len = p.row_base = p.row_extra = 0;
  // The list lives in device memory for the life of the plan, with the two
  // words of the item feed in front of it (zero between launches).
  const size_t bytes = core->host_items.size() * sizeof(uint32_t);
  constexpr size_t kFeedBytes = 16;
  void* block = nullptr;
  MUP_CUDA(cudaMalloc(&block, kFeedBytes + bytes));
  void* table = static_cast<char*>(block) + kFeedBytes;
  cudaError_t e = cudaMemset(block, 0, kFeedBytes);
  if (e == cudaSuccess) e = cudaMemcpy(table, core->host_items.data(), bytes, cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    cudaFree(block);
    return fail(MUP_ERR_CUDA, "uploading the work-item list failed: %s", cudaGetErrorString(e));
  }
  p.feed = schedule.fed ? static_cast<unsigned int*>(block) : nullptr;
  core->device_items = block;
  p.items = static_cast<const uint32_t*>(table);
  if (!list_uses_narrow_class(core->host_items)) p.flags |= mup::kFlagNoNarrowClass;
  if (const char* env = getenv("MEGA_UP_KERNEL_FLAGS")) p.flags ^= static_cast<unsigned int>(atoi(env));
  return MUP_OK;
}

// W tensor maps: box j holds the rows one CTA loads for a part of (j + 1) * 64 columns.
int encode_weight_maps(mup::GemmParams* p, const void* weight, int n, int k, int g) {
  for (int j = 0; j < mup::kNumBMaps; ++j) {
    const int rc = encode_map(&p->map_b[j], weight, k, n, k, mup::kBlockK, (j + 1) * mup::kUnit / g);
    if (rc != MUP_OK) return rc;
  }
  return MUP_OK;
}

// Launches go to the device the plan was made for: the kernel's tensor maps,
// its work-item list and (pull) its counters live there.
int check_current_device(int device, const char* what) {
  int current = -1;
  MUP_CUDA(cudaGetDevice(&current));
  if (current != device)
    return fail(MUP_ERR_BAD_ARG, "%s was made for device %d but the current device is %d; call cudaSetDevice first",
                what, device, current);
  return MUP_OK;
}

}  // namespace

// =========================================================================
// Plans
// =========================================================================

struct mup_peer_write_plan {
  PlanCore core;
  const void* last_a = nullptr;
};

struct mup_pull_plan {
  PlanCore core;
  void* workspace = nullptr;
  uint64_t workspace_bytes = 0;
  unsigned long long launches = 0;
  unsigned long long pull_warps = 0;
};

struct mup_arena {
  CUmemGenericAllocationHandle handle = 0;
  CUdeviceptr ptr = 0;
  uint64_t bytes = 0;
  int fd = -1;
  int device = 0;
  bool owner = false;
};

// =========================================================================
// Small kernels: flag barrier and layout copies
// =========================================================================

namespace {

struct FlagParams {
  uint32_t* flags[mup::kMaxPeers];
  uint32_t* status;
  unsigned long long timeout_ns;
  uint32_t epoch;
  int up;
  int rank;
};

__global__ void flag_barrier_kernel(FlagParams fp) {
  mup::grid_dep_launch();
  mup::grid_dep_wait();  // the flag vouches for everything earlier kernels of the stream wrote
  const int peer = threadIdx.x;
  if (peer >= fp.up) return;
  // Everything this GPU wrote before the barrier (including stores to peer
  // memory by earlier kernels of the stream) is ordered before the flag.
  mup::fence_acq_rel_sys();
  mup::st_release_sys(fp.flags[peer] + fp.rank, fp.epoch);
  const uint32_t* mine = fp.flags[fp.rank] + peer;
  const uint64_t t0 = mup::globaltimer_ns();
  uint32_t it = 0;
  while (static_cast<int32_t>(mup::ld_acquire_sys(mine) - fp.epoch) < 0) {
    if ((++it & 0x1fu) == 0) {
      if (mup::globaltimer_ns() - t0 > fp.timeout_ns) {
        if (fp.status != nullptr) {
          *reinterpret_cast<volatile uint32_t*>(fp.status) =
              (mup::ST_FLAG_TIMEOUT << 24) | (static_cast<uint32_t>(peer) & 0xFFFFFFu);
        }
        return;
      }
      __nanosleep(100);
    }
  }
  mup::fence_acq_rel_sys();
}

// dst row i <- src row index[i]; rows are `vecs` 16-byte vectors wide.
__global__ void gather_rows_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src,
                                   const int64_t* __restrict__ index, int64_t rows, int64_t vecs) {
  mup::grid_dep_launch();
  mup::grid_dep_wait();
  const int64_t total = rows * vecs;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += stride) {
    const int64_t row = i / vecs;
    const int64_t col = i - row * vecs;
    const int64_t srow = (index != nullptr) ? index[row] : row;
    dst[i] = src[srow * vecs + col];
  }
}

// Source-major [up, batch, seq] <-> batch-major [batch, up, seq] regroup of rows.
__global__ void regroup_rows_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, int up,
                                    int batch, int64_t seq, int64_t vecs, int to_batch_major) {
  mup::grid_dep_launch();
  mup::grid_dep_wait();
  const int64_t rows = static_cast<int64_t>(up) * batch * seq;
  const int64_t total = rows * vecs;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += stride) {
    const int64_t row = i / vecs;
    const int64_t col = i - row * vecs;
    const int64_t s = row % seq;
    const int64_t outer = row / seq;
    int64_t srow;
    if (to_batch_major) {
      const int64_t r = outer % up;  // dst row = (b*up + r)*seq + s
      const int64_t b = outer / up;
      srow = (r * batch + b) * seq + s;
    } else {
      const int64_t b = outer % batch;  // dst row = (r*batch + b)*seq + s
      const int64_t r = outer / batch;
      srow = (b * up + r) * seq + s;
    }
    dst[i] = src[srow * vecs + col];
  }
}

// Round-trip time of dependent loads: every load's address depends on the value
// before it (the buffer holds zeros), so the loads cannot overlap.
__global__ void load_latency_kernel(const unsigned long long* __restrict__ ptr, int iters,
                                    unsigned long long* __restrict__ out_ns) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const volatile unsigned long long* p = ptr;
  unsigned long long offset = 0;
  for (int i = 0; i < 16; ++i) offset = p[offset];  // warm the path (TLB, routing)
  const uint64_t t0 = mup::globaltimer_ns();
  for (int i = 0; i < iters; ++i) offset = p[offset + (static_cast<unsigned long long>(i) & 15ull) * 16ull];
  const uint64_t t1 = mup::globaltimer_ns();
  out_ns[0] = t1 - t0 + offset;  // offset is 0; keeps the chain alive
}

// The two copies with the hand-off folded in: every block waits (thread 0
// polls this rank's flags) before it touches the slots, and counts itself in
// after its last store; the last block raises the flags at the peers.
__global__ void __launch_bounds__(1024) gather_rows_synced_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src,
                                          const int64_t* __restrict__ index, int64_t rows,
                                          int64_t vecs, mup::SyncParams sp) {
  mup::grid_dep_launch();
  mup::grid_dep_wait();  // this rank's own earlier kernels (they wrote or still read what is copied here)
  // threads 0 .. up-1 poll one peer's flag each; the block proceeds on a unanimous vote
  const int handed = __syncthreads_and(mup::sync_wait_one(sp, static_cast<int>(threadIdx.x)) ? 1 : 0);
  if (handed) {
    const int64_t total = rows * vecs;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += stride) {
      const int64_t row = i / vecs;
      const int64_t col = i - row * vecs;
      const int64_t srow = (index != nullptr) ? index[row] : row;
      dst[i] = src[srow * vecs + col];
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) mup::sync_arrive_and_signal(sp);
}

__global__ void __launch_bounds__(1024) regroup_rows_synced_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src,
                                           int up, int batch, int64_t seq, int64_t vecs,
                                           int to_batch_major, mup::SyncParams sp) {
  mup::grid_dep_launch();
  mup::grid_dep_wait();  // this rank's own earlier kernels (they wrote or still read what is copied here)
  // threads 0 .. up-1 poll one peer's flag each; the block proceeds on a unanimous vote
  const int handed = __syncthreads_and(mup::sync_wait_one(sp, static_cast<int>(threadIdx.x)) ? 1 : 0);
  if (handed) {
    const int64_t rows = static_cast<int64_t>(up) * batch * seq;
    const int64_t total = rows * vecs;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += stride) {
      const int64_t row = i / vecs;
      const int64_t col = i - row * vecs;
      const int64_t s = row % seq;
      const int64_t outer = row / seq;
      int64_t srow;
      if (to_batch_major) {
        const int64_t r = outer % up;
        const int64_t b = outer / up;
        srow = (r * batch + b) * seq + s;
      } else {
        const int64_t b = outer % batch;
        const int64_t r = outer / batch;
        srow = (b * up + r) * seq + s;
      }
      dst[i] = src[srow * vecs + col];
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) mup::sync_arrive_and_signal(sp);
}

int device_sm_count() {
  // the copies run on the current device; cache its SM count per device ordinal
  static int cached[64] = {0};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 148;
  if (cached[device] == 0) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0) return 148;
    cached[device] = sms;
  }
  return cached[device];
}

// Grid of a copy that carries a hand-off: blocks of 1024 threads, at most two
// per SM, so that all of them are resident at once (every block's wait is paid
// once, concurrently) and the arrival counter sees a few hundred atomics, not
// thousands: same-address atomics take about 8 ns each, and the blocks of a
// copy all finish at about the same time.
constexpr int kSyncedCopyThreads = 1024;
int synced_copy_grid(int64_t total_vecs) {
  int64_t blocks = (total_vecs + kSyncedCopyThreads - 1) / kSyncedCopyThreads;
  const int64_t cap = static_cast<int64_t>(device_sm_count()) * 2;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

int copy_grid(int64_t total_vecs) {
  int64_t blocks = (total_vecs + 255) / 256;
  const int64_t cap = static_cast<int64_t>(device_sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

}  // namespace

// =========================================================================
// extern "C"
// =========================================================================

extern "C" {

int mup_abi_version(void) { return MUP_ABI_VERSION; }

const char* mup_last_error(void) { return g_last_error; }

int mup_device_supported(int device, int* supported) {
  if (supported == nullptr) return fail(MUP_ERR_BAD_ARG, "supported is null");
  DeviceInfo info;
  int rc = query_device(device, &info);
  if (rc != MUP_OK) return rc;
  *supported = (info.cc_major == 10) ? 1 : 0;
  return MUP_OK;
}

int mup_shape_rule(int64_t width, int up) { return shape_rule(width, up); }

int mup_peer_n_rotation(int rank, int up, int n_total, int tile_n) {
  if (up <= 0 || n_total <= 0 || tile_n <= 0 || rank < 0) return 0;
  return n_rotation(rank, up, n_total, tile_n);
}

int mup_set_max_active_ctas(int max_ctas) {
  if (max_ctas < 0) return fail(MUP_ERR_BAD_ARG, "max_ctas must be >= 0");
  g_max_ctas_option = max_ctas;
  return MUP_OK;
}

// ---------------------------------------------------------------- schedule preview

int mup_schedule_preview(int mode, int rows, int n, int k, int up, int rank, int cta_group, int slots,
                         uint32_t* items, int capacity, int* count, int* max_item_cols,
                         double* model_cycles) {
  if (mode != mup::MODE_PEER_WRITE && mode != mup::MODE_PULL) return fail(MUP_ERR_BAD_ARG, "mode must be 0 or 1");
  if (rows <= 0 || n <= 0 || k <= 0 || n % 256 || slots <= 0 || up < 1 || rank < 0 || rank >= up)
    return fail(MUP_ERR_BAD_ARG, "bad schedule arguments");
  if (cta_group < 0 || cta_group > 2) return fail(MUP_ERR_BAD_ARG, "cta_group must be 0, 1 or 2");
  const int g = (cta_group == 0) ? 2 : cta_group;
  const int m_tiles = (rows + mup::kBlockM * g - 1) / (mup::kBlockM * g);
  if (m_tiles > mup::kMaxItemMTiles || n / mup::kUnit > mup::kMaxItemNUnits)
    return fail(MUP_ERR_UNSUPPORTED, "rows=%d or n=%d exceeds the schedule's range", rows, n);
  const Schedule schedule =
      choose_schedule(mode, m_tiles, n, (k + mup::kBlockK - 1) / mup::kBlockK, up, rank, g, slots);
  if (count != nullptr) *count = static_cast<int>(schedule.items.size());
  if (max_item_cols != nullptr) *max_item_cols = schedule.max_cols;
  if (model_cycles != nullptr) *model_cycles = schedule.critical_cycles;
  if (items != nullptr) {
    const size_t copy = std::min(schedule.items.size(), static_cast<size_t>(capacity < 0 ? 0 : capacity));
    memcpy(items, schedule.items.data(), copy * sizeof(uint32_t));
  }
  return MUP_OK;
}

// ---------------------------------------------------------------- status

int mup_status_create(uint32_t** host_ptr, void** device_ptr) {
  if (host_ptr == nullptr || device_ptr == nullptr) return fail(MUP_ERR_BAD_ARG, "null output");
  void* h = nullptr;
  MUP_CUDA(cudaHostAlloc(&h, 64, cudaHostAllocMapped | cudaHostAllocPortable));
  memset(h, 0, 64);
  void* d = nullptr;
  MUP_CUDA(cudaHostGetDevicePointer(&d, h, 0));
  *host_ptr = static_cast<uint32_t*>(h);
  *device_ptr = d;
  return MUP_OK;
}

int mup_status_destroy(uint32_t* host_ptr) {
  if (host_ptr == nullptr) return MUP_OK;
  MUP_CUDA(cudaFreeHost(host_ptr));
  return MUP_OK;
}

// ---------------------------------------------------------------- arena

int mup_arena_create(int device, uint64_t bytes, mup_arena** out) {
  if (out == nullptr || bytes == 0) return fail(MUP_ERR_BAD_ARG, "bad arena arguments");
  const DriverApi& d = driver();
  if (!d.ok) return fail(MUP_ERR_DRIVER, "%s", d.error);
  MUP_CUDA(cudaSetDevice(device));
  MUP_CUDA(cudaFree(nullptr));
  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t gran = 0;
  MUP_DRV(d.mem_get_granularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED),
          "cuMemGetAllocationGranularity");
  const uint64_t size = (bytes + gran - 1) / gran * gran;
  mup_arena* a = new (std::nothrow) mup_arena();
  if (a == nullptr) return fail(MUP_ERR_BAD_ARG, "out of host memory");
  a->device = device;
  a->owner = true;
  a->bytes = size;
  CUresult r = d.mem_create(&a->handle, size, &prop, 0);
  if (r != CUDA_SUCCESS) {
    delete a;
    return driver_fail("cuMemCreate", r);
  }
  r = d.mem_address_reserve(&a->ptr, size, gran, 0, 0);
  if (r != CUDA_SUCCESS) {
    d.mem_release(a->handle);
    delete a;
    return driver_fail("cuMemAddressReserve", r);
  }
  r = d.mem_map(a->ptr, size, 0, a->handle, 0);
  if (r != CUDA_SUCCESS) {
    d.mem_address_free(a->ptr, size);
    d.mem_release(a->handle);
    delete a;
    return driver_fail("cuMemMap", r);
  }
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  r = d.mem_set_access(a->ptr, size, &acc, 1);
  if (r == CUDA_SUCCESS) {
    int fd = -1;
    r = d.mem_export(&fd, a->handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
    a->fd = fd;
  }
  if (r != CUDA_SUCCESS) {
    d.mem_unmap(a->ptr, size);
    d.mem_address_free(a->ptr, size);
    d.mem_release(a->handle);
    delete a;
    return driver_fail("cuMemSetAccess/cuMemExportToShareableHandle", r);
  }
  cudaError_t e = cudaMemset(reinterpret_cast<void*>(a->ptr), 0, size);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    mup_arena_destroy(a);
    return fail(MUP_ERR_CUDA, "zero-filling the arena failed: %s", cudaGetErrorString(e));
  }
  *out = a;
  return MUP_OK;
}

int mup_arena_import(int device, int fd, uint64_t mapped_bytes, mup_arena** out) {
  if (out == nullptr || fd < 0 || mapped_bytes == 0) return fail(MUP_ERR_BAD_ARG, "bad import arguments");
  const DriverApi& d = driver();
  if (!d.ok) return fail(MUP_ERR_DRIVER, "%s", d.error);
  MUP_CUDA(cudaSetDevice(device));
  MUP_CUDA(cudaFree(nullptr));
  mup_arena* a = new (std::nothrow) mup_arena();
  if (a == nullptr) return fail(MUP_ERR_BAD_ARG, "out of host memory");
  a->device = device;
  a->owner = false;
  a->bytes = mapped_bytes;
  CUresult r = d.mem_import(&a->handle, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                            CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  if (r != CUDA_SUCCESS) {
    delete a;
    return driver_fail("cuMemImportFromShareableHandle", r);
  }
  r = d.mem_address_reserve(&a->ptr, mapped_bytes, 0, 0, 0);
  if (r != CUDA_SUCCESS) {
    d.mem_release(a->handle);
    delete a;
    return driver_fail("cuMemAddressReserve", r);
  }
  r = d.mem_map(a->ptr, mapped_bytes, 0, a->handle, 0);
  if (r != CUDA_SUCCESS) {
    d.mem_address_free(a->ptr, mapped_bytes);
    d.mem_release(a->handle);
    delete a;
    return driver_fail("cuMemMap", r);
  }
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  r = d.mem_set_access(a->ptr, mapped_bytes, &acc, 1);
  if (r != CUDA_SUCCESS) {
    d.mem_unmap(a->ptr, mapped_bytes);
    d.mem_address_free(a->ptr, mapped_bytes);
    d.mem_release(a->handle);
    delete a;
    return driver_fail("cuMemSetAccess (is peer access available between the two GPUs?)", r);
  }
  *out = a;
  return MUP_OK;
}

int mup_arena_info(const mup_arena* arena, void** device_ptr, uint64_t* mapped_bytes, int* fd) {
  if (arena == nullptr) return fail(MUP_ERR_BAD_ARG, "arena is null");
  if (device_ptr != nullptr) *device_ptr = reinterpret_cast<void*>(arena->ptr);
  if (mapped_bytes != nullptr) *mapped_bytes = arena->bytes;
  if (fd != nullptr) *fd = arena->fd;
  return MUP_OK;
}

int mup_arena_destroy(mup_arena* arena) {
  if (arena == nullptr) return MUP_OK;
  const DriverApi& d = driver();
  if (d.ok) {
    if (arena->ptr != 0) {
      d.mem_unmap(arena->ptr, arena->bytes);
      d.mem_address_free(arena->ptr, arena->bytes);
    }
    if (arena->handle != 0) d.mem_release(arena->handle);
  }
  if (arena->owner && arena->fd >= 0) close(arena->fd);
  delete arena;
  return MUP_OK;
}

// ---------------------------------------------------------------- flags

int mup_flag_barrier(void* const* peer_flags, int up, int rank, uint32_t epoch,
                     void* status_device_ptr, uint64_t timeout_ns, void* stream) {
  if (peer_flags == nullptr || up < 1 || up > mup::kMaxPeers || rank < 0 || rank >= up)
    return fail(MUP_ERR_BAD_ARG, "bad flag barrier arguments");
  FlagParams fp;
  memset(&fp, 0, sizeof(fp));
  for (int i = 0; i < up; ++i) {
    if (peer_flags[i] == nullptr) return fail(MUP_ERR_BAD_ARG, "flag array %d is null", i);
    fp.flags[i] = static_cast<uint32_t*>(peer_flags[i]);
  }
  fp.status = static_cast<uint32_t*>(status_device_ptr);
  fp.timeout_ns = timeout_ns;
  fp.epoch = epoch;
  fp.up = up;
  fp.rank = rank;
  MUP_CUDA(launch_small(flag_barrier_kernel, 1, 32, static_cast<cudaStream_t>(stream), fp));
  return MUP_OK;
}

// ---------------------------------------------------------------- peer write

int mup_peer_write_plan_create(mup_peer_write_plan** out, int device, int rows, int n, int k, int up,
                               int rank, const void* weight, const void* bias,
                               void* const* slot_ptrs, int cta_group, void* status_device_ptr,
                               uint64_t timeout_ns) {
  if (out == nullptr || slot_ptrs == nullptr) return fail(MUP_ERR_BAD_ARG, "null argument");
  int rc = check_common(device, rows, n, k, up, rank, weight, bias, cta_group);
  if (rc != MUP_OK) return rc;
  if (shape_rule(n, up) != 0)
    return fail(MUP_ERR_BAD_ARG, "n=%d cannot be exchanged across up=%d ranks (rule %d)", n, up,
                shape_rule(n, up));
  mup_peer_write_plan* plan = new (std::nothrow) mup_peer_write_plan();
  if (plan == nullptr) return fail(MUP_ERR_BAD_ARG, "out of host memory");
  mup::GemmParams& p = plan->core.params;
  memset(&p, 0, sizeof(p));
  rc = finish_core<mup::MODE_PEER_WRITE>(&plan->core, device, rows, n, k, up, rank, cta_group);
  if (rc == MUP_OK) {
    const int g = plan->core.cta_group;
    p.shard = n / up;
    p.bias = static_cast<const __nv_bfloat16*>(bias);
    p.status = static_cast<uint32_t*>(status_device_ptr);
    p.timeout_ns = timeout_ns;
    rc = encode_weight_maps(&p, weight, n, k, g);
    for (int d = 0; d < up && rc == MUP_OK; ++d) {
      if (slot_ptrs[d] == nullptr) rc = fail(MUP_ERR_BAD_ARG, "slot pointer %d is null", d);
      if (rc == MUP_OK)
        rc = encode_map(&p.map_out[d], slot_ptrs[d], p.shard, rows, p.shard, mup::kEpiCols,
                        mup::kEpiRows);
    }
  }
  if (rc != MUP_OK) {
    delete plan;
    return rc;
  }
  *out = plan;
  return MUP_OK;
}

int mup_peer_write_launch(mup_peer_write_plan* plan, const void* a, void* stream) {
  if (plan == nullptr || a == nullptr) return fail(MUP_ERR_BAD_ARG, "null argument");
  mup::GemmParams& p = plan->core.params;
  int rc_device = check_current_device(plan->core.device, "this peer-write plan");
  if (rc_device != MUP_OK) return rc_device;
  if (a != plan->last_a) {
    int rc = encode_map(&p.map_a, a, p.K, p.M, p.K, mup::kBlockK, mup::kBlockM);
    if (rc != MUP_OK) return rc;
    plan->last_a = a;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (plan->core.cta_group == 2)
    return launch_kernel<2, mup::MODE_PEER_WRITE>(p, plan->core.grid, s);
  return launch_kernel<1, mup::MODE_PEER_WRITE>(p, plan->core.grid, s);
}

int mup_peer_write_launch_synced(mup_peer_write_plan* plan, const void* a, void* stream,
                                 mup_sync* sync) {
  if (plan == nullptr) return fail(MUP_ERR_BAD_ARG, "plan is null");
  int rc = fill_sync(&plan->core.params.sync, sync, static_cast<unsigned long long>(plan->core.grid));
  if (rc != MUP_OK) return rc;
  rc = mup_peer_write_launch(plan, a, stream);
  memset(&plan->core.params.sync, 0, sizeof(plan->core.params.sync));
  return rc;
}

int mup_peer_write_plan_info(const mup_peer_write_plan* plan, int* grid_ctas, int* cta_group,
                             int* n_rotation_out, int* smem_bytes, int* tile_n) {
  if (plan == nullptr) return fail(MUP_ERR_BAD_ARG, "plan is null");
  if (tile_n != nullptr) *tile_n = plan->core.params.max_item_cols;
  if (grid_ctas != nullptr) *grid_ctas = plan->core.grid;
  if (cta_group != nullptr) *cta_group = plan->core.cta_group;
  // first column of the first work item, in 256-column blocks
  if (n_rotation_out != nullptr)
    *n_rotation_out = plan->core.host_items.empty()
                          ? 0
                          : static_cast<int>((plan->core.host_items[0] >> 14) & 0xFFFu) * mup::kUnit / mup::kBlockN;
  if (smem_bytes != nullptr) *smem_bytes = plan->core.smem_bytes;
  return MUP_OK;
}

int mup_peer_write_plan_set_trace(mup_peer_write_plan* plan, void* trace_buffer) {
  if (plan == nullptr) return fail(MUP_ERR_BAD_ARG, "plan is null");
  if (reinterpret_cast<uintptr_t>(trace_buffer) % 8) return fail(MUP_ERR_BAD_ARG, "trace buffer must be 8-byte aligned");
  plan->core.params.trace = static_cast<unsigned long long*>(trace_buffer);
  return MUP_OK;
}

int mup_peer_write_plan_destroy(mup_peer_write_plan* plan) {
  delete plan;
  return MUP_OK;
}

// ---------------------------------------------------------------- pull

int mup_pull_ticket_shape(int shard_elems, int* rows, int* segments) {
  if (shard_elems <= 0 || shard_elems % 8) return fail(MUP_ERR_BAD_ARG, "shard must be a positive multiple of 8 elements");
  mup::GemmParams p;
  memset(&p, 0, sizeof(p));
  p.shard = shard_elems;
  p.up = 1;
  set_pull_geometry(p, 1);
  if (rows != nullptr) *rows = p.pull_rows;
  if (segments != nullptr) *segments = p.pull_segs;
  return MUP_OK;
}

uint64_t mup_pull_workspace_bytes(int rows) {
  if (rows <= 0) return 0;
  const uint64_t panels = (static_cast<uint64_t>(rows) + mup::kBlockM - 1) / mup::kBlockM;
  // [0] ticket cursor (on its own 128-byte line), [16 ..] one claim word per pull warp, then
  // the per-panel ready counts
  return (16 + mup::kPullClaimWords + panels) * sizeof(unsigned long long);
}

int mup_pull_plan_create(mup_pull_plan** out, int device, int rows, int n, int k, int up, int rank,
                         int peer_rows, const void* weight, const void* bias,
                         void* const* peer_arena_ptrs, void* dy, void* out_buf, void* workspace,
                         int cta_group, void* status_device_ptr, uint64_t timeout_ns) {
  if (out == nullptr || peer_arena_ptrs == nullptr || dy == nullptr || out_buf == nullptr ||
      workspace == nullptr)
    return fail(MUP_ERR_BAD_ARG, "null argument");
  int rc = check_common(device, rows, n, k, up, rank, weight, bias, cta_group);
  if (rc != MUP_OK) return rc;
  if (shape_rule(k, up) != 0)
    return fail(MUP_ERR_BAD_ARG, "k=%d cannot be exchanged across up=%d ranks (rule %d)", k, up,
                shape_rule(k, up));
  if (peer_rows < rows) return fail(MUP_ERR_BAD_ARG, "peer_rows=%d < rows=%d", peer_rows, rows);
  if (reinterpret_cast<uintptr_t>(workspace) % 128)
    return fail(MUP_ERR_BAD_ARG, "workspace must be 128-byte aligned");
  mup_pull_plan* plan = new (std::nothrow) mup_pull_plan();
  if (plan == nullptr) return fail(MUP_ERR_BAD_ARG, "out of host memory");
  mup::GemmParams& p = plan->core.params;
  memset(&p, 0, sizeof(p));
  rc = finish_core<mup::MODE_PULL>(&plan->core, device, rows, n, k, up, rank, cta_group);
  if (rc == MUP_OK) {
    const int g = plan->core.cta_group;
    p.shard = k / up;
    p.bias = static_cast<const __nv_bfloat16*>(bias);
    p.status = static_cast<uint32_t*>(status_device_ptr);
    p.timeout_ns = timeout_ns;
    p.dy = static_cast<__nv_bfloat16*>(dy);
    p.peer_rows = peer_rows;
    unsigned long long* ws = static_cast<unsigned long long*>(workspace);
    p.cursor = ws;
    p.claimed = ws + 16;
    p.ready = ws + 16 + mup::kPullClaimWords;
    set_pull_geometry(p, rows);
    for (int i = 0; i < up && rc == MUP_OK; ++i) {
      if (peer_arena_ptrs[i] == nullptr || reinterpret_cast<uintptr_t>(peer_arena_ptrs[i]) % 16)
        rc = fail(MUP_ERR_BAD_ARG, "peer arena pointer %d is null or not 16-byte aligned", i);
      p.peers[i] = static_cast<const __nv_bfloat16*>(peer_arena_ptrs[i]);
    }
    if (rc == MUP_OK) rc = encode_map(&p.map_a, dy, k, rows, k, mup::kBlockK, mup::kBlockM);
    if (rc == MUP_OK) rc = encode_weight_maps(&p, weight, n, k, g);
    if (rc == MUP_OK)
      rc = encode_map(&p.map_out[0], out_buf, n, rows, n, mup::kEpiCols, mup::kEpiRows);
    plan->workspace = workspace;
    plan->workspace_bytes = mup_pull_workspace_bytes(rows);
    plan->pull_warps = static_cast<unsigned long long>(plan->core.grid) * mup::kPullWarps;
    p.pull_stride = static_cast<int>(plan->pull_warps);
    if (p.pull_stride > mup::kPullClaimWords) p.claimed = nullptr;  // more pull warps than claim words: no stealing
  }
  if (rc != MUP_OK) {
    delete plan;
    return rc;
  }
  *out = plan;
  return MUP_OK;
}

int mup_pull_launch(mup_pull_plan* plan, void* stream) {
  if (plan == nullptr) return fail(MUP_ERR_BAD_ARG, "plan is null");
  mup::GemmParams& p = plan->core.params;
  int rc_device = check_current_device(plan->core.device, "this pull plan");
  if (rc_device != MUP_OK) return rc_device;
  // Tickets are drawn in chunks; every pull warp draws exactly one chunk past
  // the end before it stops, so a launch advances the cursor by chunks + pull_warps.
  const unsigned long long block = plan->pull_warps * mup::kPullChunk;
  const unsigned long long chunks =
      (static_cast<unsigned long long>(p.total_tickets) + block - 1) / block * plan->pull_warps;
  // Chunks 0 .. pull_warps-1 are pre-assigned (one per pull warp), the cursor
  // hands out chunks pull_warps .. chunks-1 and one miss per warp.
  const unsigned long long drawn = (chunks > plan->pull_warps ? chunks - plan->pull_warps : 0ull);
  p.epoch1 = plan->launches + 1;
  p.cursor_base = plan->launches * (drawn + plan->pull_warps);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int rc = (plan->core.cta_group == 2) ? launch_kernel<2, mup::MODE_PULL>(p, plan->core.grid, s)
                                       : launch_kernel<1, mup::MODE_PULL>(p, plan->core.grid, s);
  if (rc == MUP_OK) plan->launches += 1;
  return rc;
}

int mup_pull_launch_synced(mup_pull_plan* plan, void* stream, mup_sync* sync) {
  if (plan == nullptr) return fail(MUP_ERR_BAD_ARG, "plan is null");
  int rc = fill_sync(&plan->core.params.sync, sync, plan->pull_warps);
  if (rc != MUP_OK) return rc;
  rc = mup_pull_launch(plan, stream);
  memset(&plan->core.params.sync, 0, sizeof(plan->core.params.sync));
  return rc;
}

int mup_pull_plan_reset(mup_pull_plan* plan, void* stream) {
  if (plan == nullptr) return fail(MUP_ERR_BAD_ARG, "plan is null");
  MUP_CUDA(cudaMemsetAsync(plan->workspace, 0, plan->workspace_bytes,
                           static_cast<cudaStream_t>(stream)));
  if (plan->core.params.feed != nullptr)
    MUP_CUDA(cudaMemsetAsync(plan->core.params.feed, 0, 16, static_cast<cudaStream_t>(stream)));
  plan->launches = 0;
  return MUP_OK;
}

int mup_pull_plan_info(const mup_pull_plan* plan, int* grid_ctas, int* cta_group,
                       uint64_t* launches, int* smem_bytes, int* tile_n) {
  if (plan == nullptr) return fail(MUP_ERR_BAD_ARG, "plan is null");
  if (tile_n != nullptr) *tile_n = plan->core.params.max_item_cols;
  if (grid_ctas != nullptr) *grid_ctas = plan->core.grid;
  if (cta_group != nullptr) *cta_group = plan->core.cta_group;
  if (launches != nullptr) *launches = plan->launches;
  if (smem_bytes != nullptr) *smem_bytes = plan->core.smem_bytes;
  return MUP_OK;
}

int mup_pull_plan_set_trace(mup_pull_plan* plan, void* trace_buffer) {
  if (plan == nullptr) return fail(MUP_ERR_BAD_ARG, "plan is null");
  if (reinterpret_cast<uintptr_t>(trace_buffer) % 8) return fail(MUP_ERR_BAD_ARG, "trace buffer must be 8-byte aligned");
  plan->core.params.trace = static_cast<unsigned long long*>(trace_buffer);
  return MUP_OK;
}

int mup_pull_plan_destroy(mup_pull_plan* plan) {
  delete plan;
  return MUP_OK;
}

// ---------------------------------------------------------------- pull without allocation

}  // extern "C" (reopened below; the scratch array and its set-up are file-local)

namespace {

// Scratch of the allocation-free pull entry point: the ticket cursor (word 0),
// one claim word per pull warp (from word 16) and one ready count per 128-row
// panel behind them. It lives in the
// library's device image, so every GPU that loads the library holds these
// bytes until the process exits, and every call on a GPU shares them.
constexpr int kNoAllocMaxRows = MUP_NOALLOC_MAX_ROWS;
constexpr int kNoAllocScratchWords = 16 + mup::kPullClaimWords + kNoAllocMaxRows / mup::kBlockM;
static __device__ __align__(256) unsigned long long g_noalloc_pull_scratch[kNoAllocScratchWords];

constexpr int kNoAllocMaxDevices = 64;

struct NoAllocDevice {
  bool ready = false;
  unsigned long long* scratch = nullptr;  // device address of g_noalloc_pull_scratch on this GPU
  int sms = 0;
  int max_clusters = 0;  // co-resident 2-CTA clusters of the pull kernel
};

NoAllocDevice g_noalloc_devices[kNoAllocMaxDevices];
std::mutex g_noalloc_mutex;

// Once per device, with that device current: resolve the scratch symbol to a
// device address (in host code the array's name is only a stand-in for it)
// and raise the kernels' dynamic shared-memory limit.
int noalloc_setup(int device, const NoAllocDevice** out) {
  if (device < 0 || device >= kNoAllocMaxDevices)
    return fail(MUP_ERR_BAD_ARG, "device %d outside [0, %d)", device, kNoAllocMaxDevices);
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  NoAllocDevice& slot = g_noalloc_devices[device];
  if (!slot.ready) {
    int previous = -1;
    MUP_CUDA(cudaGetDevice(&previous));
    if (previous != device) MUP_CUDA(cudaSetDevice(device));
    void* address = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&address, g_noalloc_pull_scratch);
    int rc = MUP_OK;
    if (e != cudaSuccess || address == nullptr) {
      rc = fail(MUP_ERR_CUDA, "cudaGetSymbolAddress(scratch) failed on device %d: %s", device,
                cudaGetErrorString(e));
    }
    DeviceInfo info;
    if (rc == MUP_OK) rc = query_device(device, &info);
    if (rc == MUP_OK && info.cc_major != 10)
      rc = fail(MUP_ERR_UNSUPPORTED, "device %d has compute capability %d.x; sm_100 is required",
                device, info.cc_major);
    int ignored = 0, clusters = 0;
    if (rc == MUP_OK) rc = configure_kernel<1, mup::MODE_PULL>(&ignored);
    if (rc == MUP_OK) rc = configure_kernel<2, mup::MODE_PULL>(&clusters);
    if (previous != device) cudaSetDevice(previous);
    if (rc != MUP_OK) return rc;
    slot.scratch = static_cast<unsigned long long*>(address);
    slot.sms = info.sms;
    slot.max_clusters = clusters;
    slot.ready = true;
  }
  *out = &slot;
  return MUP_OK;
}

}  // namespace

extern "C" {

int mup_pull_gemm_noalloc(int device, int rows, int n, int k, int up, int rank, int peer_rows,
                          const void* weight, const void* bias, void* const* peer_arena_ptrs,
                          void* dy, void* out_buf, int cta_group, void* status_device_ptr,
                          uint64_t timeout_ns, void* stream) {
  if (peer_arena_ptrs == nullptr || dy == nullptr || out_buf == nullptr)
    return fail(MUP_ERR_BAD_ARG, "null argument");
  if (rows > kNoAllocMaxRows)
    return fail(MUP_ERR_BAD_ARG,
                "rows=%d exceeds MUP_NOALLOC_MAX_ROWS=%d, the capacity of the built-in scratch; "
                "use mup_pull_plan_create with a caller-provided workspace instead",
                rows, kNoAllocMaxRows);
  if (rows <= 0 || n <= 0 || k <= 0) return fail(MUP_ERR_BAD_ARG, "rows, n and k must be positive");
  if (up != 2 && up != 4 && up != 8) return fail(MUP_ERR_BAD_ARG, "up must be 2, 4 or 8, got %d", up);
  if (rank < 0 || rank >= up) return fail(MUP_ERR_BAD_ARG, "rank %d outside [0, %d)", rank, up);
  if (n % 256) return fail(MUP_ERR_BAD_ARG, "n=%d must be a multiple of 256", n);
  if (shape_rule(k, up) != 0)
    return fail(MUP_ERR_BAD_ARG, "k=%d cannot be exchanged across up=%d ranks (rule %d)", k, up,
                shape_rule(k, up));
  if (weight == nullptr) return fail(MUP_ERR_BAD_ARG, "weight is null");
  if (bias != nullptr && reinterpret_cast<uintptr_t>(bias) % 16)
    return fail(MUP_ERR_BAD_ARG, "bias must be 16-byte aligned");
  if (cta_group < 0 || cta_group > 2) return fail(MUP_ERR_BAD_ARG, "cta_group must be 0, 1 or 2");
  if (peer_rows < rows) return fail(MUP_ERR_BAD_ARG, "peer_rows=%d < rows=%d", peer_rows, rows);

  const NoAllocDevice* dev = nullptr;
  int rc = noalloc_setup(device, &dev);
  if (rc != MUP_OK) return rc;
  // The scratch address belongs to `device`; the memset and the launch below go to the current device.
  rc = check_current_device(device, "the allocation-free pull (argument `device`)");
  if (rc != MUP_OK) return rc;

  const int g = (cta_group == 0) ? 2 : cta_group;
  mup::GemmParams p;  // on the stack: nothing here touches the heap or the device allocator
  memset(&p, 0, sizeof(p));
  p.M = rows;
  p.N = n;
  p.K = k;
  p.up = up;
  p.rank = rank;
  p.shard = k / up;
  const int m_tiles = (rows + mup::kBlockM * g - 1) / (mup::kBlockM * g);
  p.k_tiles = (k + mup::kBlockK - 1) / mup::kBlockK;
  int slots = dev->sms;
  if (g == 2) {
    slots = dev->sms / 2;
    if (slots > dev->max_clusters) slots = dev->max_clusters;
    if (slots <= 0) return fail(MUP_ERR_UNSUPPORTED, "no 2-CTA cluster fits on device %d", device);
  }
  // No work-item list here (it would have to live in device memory): every M
  // tile is cut into the same row_len items, the count that the time model
  // rates best, and the kernel derives an item from its index.
  {
    const int units = n / mup::kUnit;
    const int max_units = mup::max_item_cols(g) / mup::kUnit;
    const int q_min = (units + max_units - 1) / max_units;
    int best_q = q_min;
    double best_cost = -1.0;
    ModelShape shape;
    shape.k_tiles = p.k_tiles;
    shape.g = g;
    for (int q = q_min; q <= units; ++q) {
      const long long rounds = (static_cast<long long>(m_tiles) * q + slots - 1) / slots;
      const double cost = rounds * item_cycles((units + q - 1) / q, shape);
      if (best_cost < 0.0 || cost < best_cost * 0.999) {
        best_cost = cost;
        best_q = q;
      }
    }
    p.items = nullptr;
    p.row_len = best_q;
    p.row_base = units / best_q;
    p.row_extra = units % best_q;
    p.num_items = m_tiles * best_q;
    p.max_item_cols = ((units + best_q - 1) / best_q) * mup::kUnit;
  }
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.status = static_cast<uint32_t*>(status_device_ptr);
  p.timeout_ns = timeout_ns;
  p.dy = static_cast<__nv_bfloat16*>(dy);
  p.peer_rows = peer_rows;
  p.cursor = dev->scratch;
  p.claimed = dev->scratch + 16;
  p.ready = dev->scratch + 16 + mup::kPullClaimWords;
  p.epoch1 = 1;       // the scratch is cleared below, so every call is "the first launch"
  p.cursor_base = 0;
  set_pull_geometry(p, rows);
  for (int i = 0; i < up; ++i) {
    if (peer_arena_ptrs[i] == nullptr || reinterpret_cast<uintptr_t>(peer_arena_ptrs[i]) % 16)
      return fail(MUP_ERR_BAD_ARG, "peer arena pointer %d is null or not 16-byte aligned", i);
    p.peers[i] = static_cast<const __nv_bfloat16*>(peer_arena_ptrs[i]);
  }
  rc = encode_map(&p.map_a, dy, k, rows, k, mup::kBlockK, mup::kBlockM);
  if (rc == MUP_OK) rc = encode_weight_maps(&p, weight, n, k, g);
  if (rc == MUP_OK) rc = encode_map(&p.map_out[0], out_buf, n, rows, n, mup::kEpiCols, mup::kEpiRows);
  if (rc != MUP_OK) return rc;

  const int grid = (p.num_items < slots ? p.num_items : slots) * g;

  p.pull_stride = grid * mup::kPullWarps;
  if (p.pull_stride > mup::kPullClaimWords) p.claimed = nullptr;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // The array keeps the previous call's counts: the cursor and the ready
  // counts of the panels this call uses must start at zero.
  const size_t panels = (static_cast<size_t>(rows) + mup::kBlockM - 1) / mup::kBlockM;
  MUP_CUDA(cudaMemsetAsync(dev->scratch, 0, (16 + mup::kPullClaimWords + panels) * sizeof(unsigned long long), s));
  return (g == 2) ? launch_kernel<2, mup::MODE_PULL>(p, grid, s)
                  : launch_kernel<1, mup::MODE_PULL>(p, grid, s);
}

// ---------------------------------------------------------------- copies

int mup_gather_rows(void* dst, const void* src, const int64_t* index, int64_t rows,
                    int64_t row_elems, void* stream) {
  if (dst == nullptr || src == nullptr || rows <= 0 || row_elems <= 0 || row_elems % 8)
    return fail(MUP_ERR_BAD_ARG, "bad gather arguments (row_elems must be a multiple of 8)");
  if (reinterpret_cast<uintptr_t>(dst) % 16 || reinterpret_cast<uintptr_t>(src) % 16)
    return fail(MUP_ERR_BAD_ARG, "gather buffers must be 16-byte aligned");
  const int64_t vecs = row_elems / 8;
  MUP_CUDA(launch_small(gather_rows_kernel, copy_grid(rows * vecs), 256, static_cast<cudaStream_t>(stream),
                        static_cast<uint4*>(dst), static_cast<const uint4*>(src), index, rows, vecs));
  return MUP_OK;
}

int mup_gather_rows_synced(void* dst, const void* src, const int64_t* index, int64_t rows,
                           int64_t row_elems, void* stream, mup_sync* sync) {
  if (dst == nullptr || src == nullptr || rows <= 0 || row_elems <= 0 || row_elems % 8)
    return fail(MUP_ERR_BAD_ARG, "bad gather arguments (row_elems must be a multiple of 8)");
  if (reinterpret_cast<uintptr_t>(dst) % 16 || reinterpret_cast<uintptr_t>(src) % 16)
    return fail(MUP_ERR_BAD_ARG, "gather buffers must be 16-byte aligned");
  const int64_t vecs = row_elems / 8;
  const int grid = synced_copy_grid(rows * vecs);
  mup::SyncParams sp;
  int rc = fill_sync(&sp, sync, static_cast<unsigned long long>(grid));
  if (rc != MUP_OK) return rc;
  MUP_CUDA(launch_small(gather_rows_synced_kernel, grid, kSyncedCopyThreads, static_cast<cudaStream_t>(stream),
                        static_cast<uint4*>(dst), static_cast<const uint4*>(src), index, rows, vecs, sp));
  return MUP_OK;
}

int mup_regroup_rows_synced(void* dst, const void* src, int up, int batch, int64_t seq,
                            int64_t row_elems, int to_batch_major, void* stream, mup_sync* sync) {
  if (dst == nullptr || src == nullptr || up <= 0 || batch <= 0 || seq <= 0 || row_elems <= 0 ||
      row_elems % 8)
    return fail(MUP_ERR_BAD_ARG, "bad regroup arguments (row_elems must be a multiple of 8)");
  if (reinterpret_cast<uintptr_t>(dst) % 16 || reinterpret_cast<uintptr_t>(src) % 16)
    return fail(MUP_ERR_BAD_ARG, "regroup buffers must be 16-byte aligned");
  const int64_t vecs = row_elems / 8;
  const int64_t total = static_cast<int64_t>(up) * batch * seq * vecs;
  const int grid = synced_copy_grid(total);
  mup::SyncParams sp;
  int rc = fill_sync(&sp, sync, static_cast<unsigned long long>(grid));
  if (rc != MUP_OK) return rc;
  MUP_CUDA(launch_small(regroup_rows_synced_kernel, grid, kSyncedCopyThreads, static_cast<cudaStream_t>(stream),
                        static_cast<uint4*>(dst), static_cast<const uint4*>(src), up, batch, seq, vecs,
                        to_batch_major, sp));
  return MUP_OK;
}

int mup_probe_load_latency(const void* zeros, int iters, uint64_t* out_ns, void* stream) {
  if (zeros == nullptr || out_ns == nullptr || iters <= 0)
    return fail(MUP_ERR_BAD_ARG, "bad latency probe arguments");
  if (reinterpret_cast<uintptr_t>(zeros) % 8 || reinterpret_cast<uintptr_t>(out_ns) % 8)
    return fail(MUP_ERR_BAD_ARG, "latency probe buffers must be 8-byte aligned");
  load_latency_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const unsigned long long*>(zeros), iters, reinterpret_cast<unsigned long long*>(out_ns));
  MUP_CUDA(cudaGetLastError());
  return MUP_OK;
}

int mup_regroup_rows(void* dst, const void* src, int up, int batch, int64_t seq, int64_t row_elems,
                     int to_batch_major, void* stream) {
  if (dst == nullptr || src == nullptr || up <= 0 || batch <= 0 || seq <= 0 || row_elems <= 0 ||
      row_elems % 8)
    return fail(MUP_ERR_BAD_ARG, "bad regroup arguments (row_elems must be a multiple of 8)");
  if (reinterpret_cast<uintptr_t>(dst) % 16 || reinterpret_cast<uintptr_t>(src) % 16)
    return fail(MUP_ERR_BAD_ARG, "regroup buffers must be 16-byte aligned");
  const int64_t vecs = row_elems / 8;
  const int64_t total = static_cast<int64_t>(up) * batch * seq * vecs;
  MUP_CUDA(launch_small(regroup_rows_kernel, copy_grid(total), 256, static_cast<cudaStream_t>(stream),
                        static_cast<uint4*>(dst), static_cast<const uint4*>(src), up, batch, seq, vecs,
                        to_batch_major));
  return MUP_OK;
}

}  // extern "C"
