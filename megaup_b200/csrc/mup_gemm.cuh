// Persistent, warp-specialised tcgen05 BF16 GEMM  out = bf16(A @ W^T + bias)
// shared by the two fused Ulysses exchange operators:
//
//   MODE_PEER_WRITE  A is local; every 32x64 output sub-tile is TMA-stored
//                    straight into the slot of the rank that owns those
//                    columns (replaces linear + permute + all_to_all).
//   MODE_PULL        pull warps copy every peer's head shard of each row
//                    into the dense local input `dy` while the MMA warps
//                    already consume finished 128-row panels (replaces
//                    all_to_all + permute + linear).
//
// Work items. The output is cut into items of 128*G rows by 64..512 columns
// (a multiple of 64), listed by the host in the order they are consumed; CTA
// (pair) c runs items c, c + #clusters, ... , or the CTAs draw the items from
// the list as they become free (the item feed, below). An item wider than 256 columns is
// computed as two parts that share every A tile: each K step loads A once and
// feeds it to two accumulators, so a 512-wide item moves 48 KiB per CTA and
// 1024 tensor cycles where two 256-wide tiles move 64 KiB. On this GPU the
// delivery of operands from L2 (about 12 TB/s over all SMs), not the tensor
// pipe, bounds 256-wide tiles at full clock; wide items bring the demand under
// that limit. A part is one accumulator of at most 256 FP32 columns in TMEM;
// the two 256-column halves of TMEM form a ring of accumulator slots that the
// parts of consecutive items take in turn, so the epilogue of a one-part item
// overlaps the K loop of the next item. A two-part item owns both slots: the
// next item's K loop waits for its epilogue, which is why the host uses wide
// items only for long K (the WIDE = false instantiation has no code for them).
//
// G = 1 runs one CTA per item (tcgen05 cta_group::1); G = 2 pairs two CTAs of a
// cluster on 256 rows (cta_group::2): each CTA loads its own 128 rows of A and
// its own half of every W box, so no load is ever multicast.
//
// The FP32 accumulator of an output element is a single TMEM cell that
// receives the K products in ascending order, 16 at a time; bias is added in
// FP32 and the sum is rounded to BF16 once. Nothing about the schedule (item
// widths, which SM runs which item, the order of items) changes that order, so
// every schedule gives the same bits.
//
// The kernel is launched with programmatic stream serialization: it lets its
// successor be scheduled at entry and waits for its predecessor after its own
// set-up.
//
// Warp roles (192 threads, 384 in pull mode):
//   warp 0      TMA producer (one elected lane)
//   warp 1      TMEM allocation + MMA issue (warp-uniform loop, one elected lane issues; leader CTA)
//   warps 2-5   epilogue; warp w owns TMEM lanes 32*(w%4) .. +31
//   warps 6-11  (pull mode) peer -> dy copy workers
//
// Every wait is bounded. A role that gives up records a code in *status,
// raises the CTA's abort flag so the other roles give up too, and all roles
// meet at the final barrier where TMEM is released.
#pragma once

#include "mup_ptx.cuh"
#include "mup_sync.cuh"

namespace mup {

constexpr int kBlockM = 128;
constexpr int kBlockN = 256;          // columns of one accumulator slot (half of TMEM)
constexpr int kBlockK = 64;           // K extent of one TMA box (128 bytes, the swizzle span)
constexpr int kUmmaK = 16;
constexpr int kMaxPeers = 8;
constexpr int kAccStages = 2;
constexpr int kTmemCols = 512;
constexpr int kEpiCols = 64;        // columns per epilogue sub-tile (128 bytes) = schedule granularity
constexpr int kEpiRows = 32;        // rows per epilogue warp
constexpr int kEpiBufBytes = kEpiRows * kEpiCols * 2;  // 4096
constexpr int kEpiBufs = 2;
constexpr int kUnit = kEpiCols;       // item widths and offsets are multiples of this
constexpr int kMaxItemUnits = 8;      // 512 columns: both accumulator slots
constexpr int kNumBMaps = 4;          // W boxes for parts of 64, 128, 192 and 256 columns
#ifndef MUP_PULL_MAX_VECS
#define MUP_PULL_MAX_VECS 512
#endif
constexpr int kPullMaxVecs = MUP_PULL_MAX_VECS;  // 16-byte vectors per pull ticket (one batch of peer loads per warp)
constexpr int kPullUnroll = kPullMaxVecs / 32;
constexpr int kFeedDepth = 16;        // entries of the item feed in shared memory (a power of two)
#ifndef MUP_PULL_WARPS
#define MUP_PULL_WARPS 6
#endif
constexpr int kPullWarps = MUP_PULL_WARPS;  // pull workers per CTA (warps 6 .. 6 + kPullWarps - 1)
constexpr int kPullChunk = 8;         // tickets drawn per atomic
constexpr int kPullClaimWords = 1024; // one claim word per pull warp of the grid (148 SMs x 6 = 888)

constexpr int MODE_PEER_WRITE = 0;
constexpr int MODE_PULL = 1;

// Device status codes (upper byte of the status word).
constexpr uint32_t ST_OK = 0;
constexpr uint32_t ST_PRODUCER_SLOT_TIMEOUT = 1;
constexpr uint32_t ST_MMA_FULL_TIMEOUT = 2;
constexpr uint32_t ST_MMA_ACC_TIMEOUT = 3;
constexpr uint32_t ST_EPILOGUE_TIMEOUT = 4;
constexpr uint32_t ST_PULL_READY_TIMEOUT = 5;
constexpr uint32_t ST_SMEM_MISALIGNED = 6;
constexpr uint32_t ST_FLAG_TIMEOUT = 7;
constexpr uint32_t ST_ITEM_FEED_TIMEOUT = 8;

// Shared-memory plan. The widest item of a launch fixes the size and with it
// the number of pipeline stages, so the layout keeps a fixed 192 KiB stage
// area and room for the largest stage count.
constexpr int kMaxStages = 8;
constexpr int kStageAreaBytes = 196608;
template <int G>
struct GemmCfg {
  static constexpr int kABytes = kBlockM * kBlockK * 2;         // 16 KB
  static constexpr int kOffEpi = kStageAreaBytes;
  static constexpr int kOffBias = kOffEpi + 4 * kEpiBufs * kEpiBufBytes;
  static constexpr int kOffBar = kOffBias + 4 * kEpiCols * 4;
  // full[kMaxStages], empty[kMaxStages], acc_full[2], acc_empty[2]
  static constexpr int kNumBars = 2 * kMaxStages + 2 * kAccStages;
  static constexpr int kOffTmemSlot = kOffBar + kNumBars * 8;
  static constexpr int kOffAbort = kOffTmemSlot + 4;
  static constexpr int kOffFeed = kOffAbort + 4;                // kFeedDepth 64-bit words (item feed)
  static constexpr int kSmemBytes = kOffFeed + kFeedDepth * 8 + 56;  // small pad
  static constexpr int kUmmaM = kBlockM * G;
};

// Widest item a CTA grouping can run: a lone CTA loads all W rows of an item
// itself, so two parts would not leave room for enough stages.
__host__ __device__ constexpr int max_item_cols(int g) { return g == 2 ? kMaxItemUnits * kUnit : kBlockN; }
// W rows one CTA loads per K step for `cols` output columns, bytes of a stage, number of stages.
__host__ __device__ constexpr int tile_b_rows(int cols, int g) { return cols / g; }
__host__ __device__ constexpr int tile_stage_bytes(int cols, int g) {
  return kBlockM * kBlockK * 2 + tile_b_rows(cols, g) * kBlockK * 2;
}
__host__ __device__ constexpr int tile_stages(int cols, int g) {
  return kStageAreaBytes / tile_stage_bytes(cols, g) > kMaxStages
             ? kMaxStages
             : kStageAreaBytes / tile_stage_bytes(cols, g);
}

// Stage geometry is chosen per item from three classes, by the item's width: up
// to 128 columns (8 stages of 24 KiB for a CTA pair), up to 256 (6 of 32 KiB)
// and up to 512 (4 of 48 KiB). Narrow items (the cut-up last round of a list)
// thus keep as many K steps in flight as the stage area allows, whatever the
// widest item of the launch is. When consecutive items of a CTA differ in class
// the TMA producer lets the pipeline drain (every stage consumed) and both
// sides restart at stage 0; which phase of a stage's barriers comes next is
// kept per stage, one bit each, so the ring may change its length.
__host__ __device__ constexpr int stage_class_cols(int cols, bool narrow_class = true) {
  return (narrow_class && cols <= 2 * kUnit) ? 2 * kUnit : (cols <= kBlockN ? kBlockN : kMaxItemUnits * kUnit);
}

// A work item as the host lists it: 14 bits M tile, 12 bits first column / 64, 3 bits (columns / 64 - 1).
__host__ __device__ constexpr uint32_t encode_item(int m_idx, int n0_units, int w_units) {
  return static_cast<uint32_t>(m_idx) | (static_cast<uint32_t>(n0_units) << 14) |
         (static_cast<uint32_t>(w_units - 1) << 26);
}
constexpr uint32_t kNoItem = 0xFFFFFFFFu;  // a list entry without work (the CTA pair sits this round out)
constexpr int kMaxItemMTiles = 1 << 14;
constexpr int kMaxItemNUnits = 1 << 12;

struct GemmParams {
  CUtensorMap map_a;                 // A  [M, K]   box 64 x 128
  CUtensorMap map_b[kNumBMaps];      // W  [N, K]   box 64 x ((j + 1) * 64 / G): this CTA's rows of a part of (j + 1) * 64 columns
  CUtensorMap map_out[kMaxPeers];    // peer-write: [rows, shard] slot in peer p; pull: [0] = out [M, N]
  const __nv_bfloat16* bias;         // nullptr when absent
  uint32_t* status;                  // error word (host-visible)
  unsigned long long timeout_ns;
  int M, N, K;
  int shard;                         // exchanged columns per rank
  int up, rank;
  int k_tiles;
  // Schedule: `items` lists the work items in consumption order. Without a list
  // (nullptr) every M tile is cut alike: row_len items, the first row_extra of
  // them row_base + 1 units wide and the rest row_base units.
  const uint32_t* items;
  int num_items;
  // Item feed (nullptr: CTA (pair) c runs items c, c + grid, ... of the list).
  // feed[0]: the next list position to hand out; feed[1]: CTAs (pairs) that
  // have finished. Both are zero between launches: the last one out clears them.
  unsigned int* feed;
  int row_len, row_base, row_extra;
  int max_item_cols;                 // widest item: fixes the stage size
  // pull mode only
  const __nv_bfloat16* peers[kMaxPeers];  // staged arenas [up(dest), peer_rows, shard]
  __nv_bfloat16* dy;                 // dense pulled input [M, K]
  unsigned long long* ready;         // [ceil(M/128)] monotonically increasing ticket counts
  unsigned long long* cursor;        // monotonically increasing cursor, in chunks of kPullChunk tickets
  unsigned long long* claimed;       // [pull_stride] launch ordinal that claimed a pull warp's pre-assigned first chunk (nullptr: no stealing)
  unsigned long long epoch1;         // launch ordinal, 1-based
  unsigned long long cursor_base;    // cursor value that means "chunk 0" for this launch
  int peer_rows;
  int total_tickets;
  int pull_stride;                   // pull warps in the grid: distance between the tickets of a chunk
  int pull_rows;                     // rows per pull ticket: a power of two <= 16 with pull_rows * shard / 8 <= kPullMaxVecs
  int pull_segs;                     // column segments per shard row (> 1 only when one row exceeds a ticket; then pull_rows = 1)
  int pull_seg_vecs;                 // 16-byte vectors per segment
  int pull_up_shift;                 // log2(up)
  int pull_panel_shift;              // log2(128 / pull_rows)
  unsigned int pull_pace_ns;         // the i-th pull warp of the grid issues its first ticket i * pace ns late (0: at once)
  unsigned int flags;                // tuning switches (kFlag*)
  unsigned long long* trace;         // optional [grid][16] cycle counters (nullptr: off)
  SyncParams sync;                   // slot hand-off folded into this launch (flags[0] == nullptr: none)
};

// Per-CTA trace slots (SM cycles unless noted), written when GemmParams::trace is set.
constexpr int kTraceStart = 0;        // clock64 at kernel entry
constexpr int kTraceEnd = 1;          // clock64 after the last role finished
constexpr int kTraceMmaWaitFull = 2;  // MMA thread waiting for operands (TMA behind)
constexpr int kTraceMmaWaitAcc = 3;   // MMA thread waiting for a free accumulator (epilogue behind)
constexpr int kTraceProdWait = 4;     // TMA producer waiting for a free stage (MMA behind: the good case)
constexpr int kTraceEpiWait = 5;      // epilogue warp 2 waiting for a finished accumulator
constexpr int kTraceNsStart = 6;      // %globaltimer at entry
constexpr int kTraceNsEnd = 7;        // %globaltimer at exit
constexpr int kTracePullEndNs = 8;    // %globaltimer when this CTA's pull workers ran out of tickets
constexpr int kTracePullTickets = 9;  // tickets copied by this CTA's pull workers
constexpr int kTraceGateFirstNs = 10; // ns from kernel entry until the producer's first panel gate opened
constexpr int kTraceGateCycles = 11;  // producer cycles spent at panel gates
constexpr int kTraceSetupNs = 12;     // ns from kernel entry until the predecessor kernel had completed (set-up done)
constexpr int kTracePullFirstNs = 13; // ns from kernel entry until the first pull warp had stored its first ticket
constexpr int kTraceFirstMmaNs = 14;  // ns from kernel entry until the first operands had landed (first MMA)
constexpr int kTraceItems = 15;       // work items this CTA (pair) ran
constexpr int kTraceSlots = 16;

constexpr unsigned int kFlagNoL2Hints = 8u;     // tuning: drop the L2 hints (W loads evict-last, output stores evict-first)
constexpr unsigned int kFlagSplitCommit = 1u;  // G=2: one commit per CTA of the pair instead of one for both
constexpr unsigned int kFlagSeparateIssue = 2u;  // tuning: poll, MMAs and commit as separate statements (the slower issue loop)
constexpr unsigned int kFlagPullExtraFence = 16u;  // tuning: an explicit fence.acq_rel.gpu before every release of a ready count
constexpr unsigned int kFlagSpinWaits = 256u;  // tuning: the TMA producer and the MMA warp poll their barriers with test_wait
// Items of at most 128 columns use the 256-column stage geometry. The host sets
// it for every list that also has wider items: changing the geometry drains
// the pipeline, which cost more (0.7-1.0 us on 4096 x 5120 x 5120) than two
// more stages gain for one short round of narrow items.
constexpr unsigned int kFlagNoNarrowClass = 128u;
constexpr unsigned int kFlagNoPartSkew = 64u;   // tuning: two-accumulator items without the skew between their parts
constexpr unsigned int kFlagNoWPrefetch = 32u;  // tuning: pull mode, do not load W ahead of a closed panel gate

// The first role of a CTA that gives up records why; roles that give up because
// the abort flag is already up leave the recorded cause alone.
__device__ __forceinline__ void report_status(const GemmParams& p, volatile uint32_t* abort_flag,
                                              uint32_t code, uint32_t detail) {
  const bool first = (*abort_flag == 0u);
  *abort_flag = 1u;
  if (first && p.status != nullptr) {
    *reinterpret_cast<volatile uint32_t*>(p.status) = (code << 24) | (detail & 0xFFFFFFu);
  }
}

// ---------------------------------------------------------------------------
// Pull tickets. Ticket t = (row group, source rank rotated from this rank,
// column segment): pull_rows rows of one peer shard (or one segment of a single
// row when a row alone exceeds a ticket), at most kPullMaxVecs 16-byte vectors.
// ---------------------------------------------------------------------------
struct PullTicket {
  const __nv_bfloat16* src;
  __nv_bfloat16* dst;
  int nvec;
  int panel;  // the 128-row panel the ticket belongs to
};

// Ticket numbers fit 32 bits (the host checks). With one segment per shard row
// (shards of at most 4096 columns, the common case) a row group holds `up`
// tickets and up is a power of two, so the split is a shift and a mask.
__device__ __forceinline__ PullTicket pull_ticket_geometry(const GemmParams& p, uint32_t t) {
  const int vec_per_row = p.shard >> 3;
  int grp, seg, hop;
  if (p.pull_segs == 1) {
    grp = static_cast<int>(t >> p.pull_up_shift);
    hop = static_cast<int>(t & static_cast<uint32_t>(p.up - 1));
    seg = 0;
  } else {
    const uint32_t per_group = static_cast<uint32_t>(p.up * p.pull_segs);
    grp = static_cast<int>(t / per_group);
    const int within = static_cast<int>(t - static_cast<uint32_t>(grp) * per_group);
    hop = within / p.pull_segs;
    seg = within - hop * p.pull_segs;
  }
  int src_rank = hop + p.rank + 1;
  if (src_rank >= p.up) src_rank -= p.up;
  const int r0 = grp * p.pull_rows;
  int nrows = p.M - r0;
  nrows = nrows > p.pull_rows ? p.pull_rows : nrows;
  const int v0 = seg * p.pull_seg_vecs;
  PullTicket k;
  if (p.pull_segs > 1) {
    k.nvec = vec_per_row - v0;
    k.nvec = k.nvec > p.pull_seg_vecs ? p.pull_seg_vecs : k.nvec;
  } else {
    k.nvec = nrows * vec_per_row;  // <= kPullMaxVecs
  }
  k.src = p.peers[src_rank] + (static_cast<size_t>(p.rank) * p.peer_rows + r0) * static_cast<size_t>(p.shard) + v0 * 8;
  k.dst = p.dy + static_cast<size_t>(r0) * p.K + static_cast<size_t>(src_rank) * p.shard + v0 * 8;
  k.panel = grp >> p.pull_panel_shift;  // pull_rows is a power of two: 128 / pull_rows groups per panel
  return k;
}

// The rows of a ticket follow each other in the peer's staged shard, so lane l's
// u-th vector is simply vector u * 32 + l of a contiguous block.
__device__ __forceinline__ void pull_ticket_load(const PullTicket& k, int lane, uint4 (&regs)[kPullUnroll]) {
#pragma unroll
  for (int u = 0; u < kPullUnroll; ++u) {
    const int vidx = u * 32 + lane;
    if (vidx < k.nvec) regs[u] = ld_stream_v4(k.src + static_cast<size_t>(vidx) * 8);
  }
}

// In dy the rows are K elements apart. (row, column vector) of lane l's first
// vector is the same for every ticket (`row0`, `vec0`, computed once per
// kernel); each further vector lies 32 vectors on, which wraps into the next
// row at most twice (a shard row has at least 16 vectors).
__device__ __forceinline__ void pull_ticket_store(const GemmParams& p, const PullTicket& k, int lane, int row0,
                                                  int vec0, const uint4 (&regs)[kPullUnroll]) {
  const int vec_per_row = p.shard >> 3;
  int cc = vec0;
  size_t row_off = static_cast<size_t>(row0) * p.K;
#pragma unroll
  for (int u = 0; u < kPullUnroll; ++u) {
    const int vidx = u * 32 + lane;
    if (vidx < k.nvec) *reinterpret_cast<uint4*>(k.dst + row_off + cc * 8) = regs[u];
    cc += 32;
    if (cc >= vec_per_row) {
      cc -= vec_per_row;
      row_off += p.K;
      if (cc >= vec_per_row) {
        cc -= vec_per_row;
        row_off += p.K;
      }
    }
  }
}

// Every lane's stores of the ticket precede this call (__syncwarp). The release
// orders them (cumulatively, through the warp barrier) before the count; the
// proxy fence orders them before the consumers' TMA reads.
__device__ __forceinline__ void pull_ticket_publish(const GemmParams& p, int panel, int lane) {
  if (lane == 0) {
    fence_proxy_async_global();
    if (p.flags & kFlagPullExtraFence) fence_acq_rel_gpu();
    red_release_gpu_add_u64(reinterpret_cast<uint64_t*>(p.ready + panel), 1ull);
  }
}

__host__ __device__ constexpr int kernel_threads(int mode) {
  return mode == MODE_PULL ? 192 + 32 * kPullWarps : 192;
}

// A decoded work item: `parts` accumulators of part_cols[] columns each, side by side from column n0.
struct WorkItem {
  int m_idx;
  int n0;
  int parts;
  int part_cols[2];
};

// The list entry of work item `item` (kNoItem past the end). Every role fetches
// the entry of its next item while it works on the current one, and the first
// entry before the kernel's set-up, so the fetch never sits between two items.
__device__ __forceinline__ uint32_t item_entry(const GemmParams& p, int item) {
  if (item >= p.num_items) return kNoItem;
  if (p.items != nullptr) return __ldg(p.items + item);
  const int m_idx = item / p.row_len;
  const int pos = item - m_idx * p.row_len;
  return encode_item(m_idx, pos * p.row_base + (pos < p.row_extra ? pos : p.row_extra),
                     p.row_base + (pos < p.row_extra ? 1 : 0));
}

__device__ __forceinline__ WorkItem decode_entry(uint32_t e) {
  WorkItem w;
  if (e == kNoItem) {
    w.m_idx = w.n0 = w.parts = 0;
    w.part_cols[0] = w.part_cols[1] = 0;
    return w;
  }
  const int w_units = static_cast<int>((e >> 26) & 0x7u) + 1;
  w.m_idx = static_cast<int>(e & 0x3FFFu);
  w.n0 = static_cast<int>((e >> 14) & 0xFFFu) * kUnit;
  if (w_units * kUnit <= kBlockN) {
    w.parts = 1;
    w.part_cols[0] = w_units * kUnit;
    w.part_cols[1] = 0;
  } else {
    w.parts = 2;
    w.part_cols[0] = ((w_units + 1) >> 1) * kUnit;
    w.part_cols[1] = (w_units >> 1) * kUnit;
  }
  return w;
}

// Item feed: with GemmParams::feed set, the CTAs (pairs) take their items from
// the list in the order they become free instead of in a fixed round-robin
// (the SMs do not run an item equally fast: with a fixed assignment the
// slowest CTA pair of 4096 x 5120 x 5120 took 3.5-8 % longer than the mean).
// One thread per CTA pair, the TMA producer of the leader CTA, draws the list
// position of its next item with an atomic when it starts an item and writes
// the drawn entry, tagged with the item's ordinal, into a small ring in the
// shared memory of both CTAs when it starts the next one; the other roles wait
// for their ordinal to appear. A position past the end of the list (kNoItem)
// ends every role. The ring needs no "slot free" signal: an entry is
// overwritten kFeedDepth items later, and the producer cannot be more than
// four items ahead of the slowest role (the stages hold less than one item,
// the two accumulators at most two more).
__device__ __forceinline__ void feed_publish(uint32_t ring_addr, int ordinal, uint32_t entry) {
  st_relaxed_cluster_smem_u64(ring_addr + 8u * static_cast<uint32_t>(ordinal & (kFeedDepth - 1)),
                              (static_cast<uint64_t>(static_cast<uint32_t>(ordinal) + 1u) << 32) | entry);
}

// False when the wait ran out or the CTA is giving up.
__device__ __forceinline__ bool feed_wait(uint32_t ring, int ordinal, volatile uint32_t* abort_flag,
                                          uint64_t timeout_ns, uint32_t* entry) {
  const uint32_t addr = ring + 8u * static_cast<uint32_t>(ordinal & (kFeedDepth - 1));
  const uint32_t want = static_cast<uint32_t>(ordinal) + 1u;
  uint64_t v = ld_relaxed_cluster_smem_u64(addr);
  if (static_cast<uint32_t>(v >> 32) != want) {
    const uint64_t t0 = globaltimer_ns();
    uint32_t polls = 0;
    do {
      if ((++polls & 63u) == 0u && (*abort_flag != 0u || globaltimer_ns() - t0 > timeout_ns)) return false;
      v = ld_relaxed_cluster_smem_u64(addr);
    } while (static_cast<uint32_t>(v >> 32) != want);
  }
  *entry = static_cast<uint32_t>(v);
  return true;
}

// WIDE = false is the kernel for lists whose items all have one accumulator (at
// most 256 columns): the code of the two-accumulator items is compiled out.
// Merely having that code in the kernel slowed single-accumulator items by
// 2.5 % (186.4 k against 181.6 k cycles per CTA for four rounds of 256-wide
// items), so each kind of list gets its own instantiation.
template <int G, int MODE, bool WIDE>
__global__ void __launch_bounds__(kernel_threads(MODE), 1)
fused_exchange_gemm_kernel(const __grid_constant__ GemmParams p) {
  constexpr bool kAllowWide = WIDE;
  using Cfg = GemmCfg<G>;
  extern __shared__ __align__(1024) uint8_t smem[];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = (G == 2) ? cluster_ctarank() : 0u;
  const int cluster_id = blockIdx.x / G;
  const int num_clusters = gridDim.x / G;
  const int num_items = p.num_items;

  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + Cfg::kOffBar;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kMaxStages + s); };
  auto acc_full_bar = [&](int a) { return bar_base + 8u * (2 * kMaxStages + a); };
  auto acc_empty_bar = [&](int a) { return bar_base + 8u * (2 * kMaxStages + kAccStages + a); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + Cfg::kOffTmemSlot);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + Cfg::kOffAbort);
  const uint64_t timeout_ns = p.timeout_ns;
  unsigned long long* trace = (p.trace != nullptr) ? p.trace + static_cast<size_t>(blockIdx.x) * kTraceSlots : nullptr;
  grid_dep_launch();  // the next kernel may be scheduled now; it waits for this one in its own grid_dep_wait
  if (trace != nullptr && threadIdx.x == 0) {
    trace[kTraceStart] = clock64();
    trace[kTraceNsStart] = globaltimer_ns();
  }
  const uint32_t first_entry = item_entry(p, cluster_id);  // the list is written when the plan is made
  const bool fed = p.feed != nullptr;
  const uint32_t feed_ring = smem_base + Cfg::kOffFeed;
  // Entry of this role's next item. Fixed assignment: `ahead` was fetched while
  // the previous item ran. 1: *entry is item `ordinal`; 0: no more items; -1: the
  // feed did not deliver in time.
  auto next_item = [&](int ordinal, int item, uint32_t& ahead, uint32_t* entry) -> int {
    if (!fed) {
      if (item >= num_items) return 0;
      *entry = ahead;
      ahead = item_entry(p, item + num_clusters);
      return 1;
    }
    if (!feed_wait(feed_ring, ordinal, abort_flag, timeout_ns, entry)) return -1;
    return *entry == kNoItem ? 0 : 1;
  };
  // Pull mode: every pull warp claims its pre-assigned first chunk for this
  // launch. The claim words only ever grow (launch ordinals), so the claim may
  // be made before the previous launch of the plan has completed, and its
  // latency hides behind the set-up below.
  bool own_first_chunk = true;
  if constexpr (MODE == MODE_PULL) {
    if (warp >= 6 && lane == 0 && p.claimed != nullptr) {
      const unsigned long long me = static_cast<unsigned long long>(blockIdx.x) * kPullWarps + (warp - 6);
      own_first_chunk = atomicMax(p.claimed + me, p.epoch1) < p.epoch1;
    }
  }

  // ------------------------------------------------------------------ set-up
  if (threadIdx.x == 0) {
    *abort_flag = 0u;
    if ((smem_base & 1023u) != 0u) report_status(p, abort_flag, ST_SMEM_MISALIGNED, smem_base);
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < kAccStages; ++a) {
      mbar_init(acc_full_bar(a), 1);
      mbar_init(acc_empty_bar(a), 4 * G);
    }
    for (int i = 0; i < kFeedDepth; ++i) reinterpret_cast<volatile uint64_t*>(smem + Cfg::kOffFeed)[i] = 0ull;
    fence_mbar_init();
    tma_prefetch_desc(&p.map_a);
#pragma unroll
    for (int j = 0; j < kNumBMaps; ++j) tma_prefetch_desc(&p.map_b[j]);
  }
  if (warp == 1) {
    tmem_alloc<G>(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
    tmem_relinquish<G>();
  }
  tc_fence_before_sync();
  if constexpr (G == 2) {
    __syncthreads();
    cluster_arrive_release();
    cluster_wait_acquire();
  } else {
    __syncthreads();
  }
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const bool misaligned = (*abort_flag != 0u);
  // Everything above touched only this CTA's shared memory and TMEM (and the
  // launch parameters); from here on the kernel reads what earlier kernels of
  // the stream wrote.
  grid_dep_wait();
  if (trace != nullptr && threadIdx.x == 0) trace[kTraceSetupNs] = globaltimer_ns() - trace[kTraceNsStart];

  // ------------------------------------------------------------ TMA producer
  if (warp == 0 && !misaligned) {
    if (lane == 0) {
      uint32_t stage = 0;
      uint32_t fills = 0;      // bit s: parity of the number of times stage s has been armed
      uint32_t in_flight = 0;  // stages armed so far in the current ring (saturates at its length)
      int num_stages = 0;      // current ring: length and stage size (0: nothing loaded yet)
      uint32_t stage_bytes = 0;
      bool ok = true;
      long long waited = 0;
      const uint32_t leader_full0 = (G == 2) ? mapa_cluster(full_bar(0), 0) : full_bar(0);
      const bool hints = (p.flags & kFlagNoL2Hints) == 0u;
      const uint64_t keep = l2_policy_evict_last();  // W is re-read by every round of items
      // A stage may be armed again once the MMAs of its previous use have read it:
      // the empty barrier's phase of that use has the parity of (uses - 1).
      auto empty_parity = [&](uint32_t s) { return ((fills >> s) & 1u) ^ 1u; };
      auto advance = [&](uint32_t& s) {
        if (++s == static_cast<uint32_t>(num_stages)) s = 0;
      };
      // With an item feed the leader CTA's producer is the one that draws.
      const bool drawer = fed && cta_rank == 0u;
      const uint32_t feed_ring_peer = (G == 2) ? mapa_cluster(feed_ring, 1) : 0u;
      auto draw = [&]() -> uint32_t {
        const unsigned int at = atomicAdd(p.feed, 1u);
        return at < static_cast<unsigned int>(num_items) ? __ldg(p.items + at) : kNoItem;
      };
      uint32_t ahead = drawer ? draw() : first_entry;
      for (int ordinal = 0, item = cluster_id; ok; ++ordinal, item += num_clusters) {
        uint32_t entry;
        if (drawer) {
          // `ahead` was drawn when the previous item started; everyone else learns of it now
          entry = ahead;
          feed_publish(feed_ring, ordinal, entry);
          if constexpr (G == 2) feed_publish(feed_ring_peer, ordinal, entry);
          if (entry == kNoItem) break;
          ahead = draw();
        } else {
          const int got = next_item(ordinal, item, ahead, &entry);
          if (got < 0) {
            report_status(p, abort_flag, ST_ITEM_FEED_TIMEOUT, static_cast<uint32_t>(ordinal));
            ok = false;
          }
          if (got <= 0) break;
        }
        const WorkItem w = decode_entry(entry);
        if (w.parts == 0) continue;
        const int panel = w.m_idx * G + static_cast<int>(cta_rank);
        const int a_row0 = panel * kBlockM;
        const int item_cols = w.part_cols[0] + w.part_cols[1];
        const uint32_t item_bytes = static_cast<uint32_t>(tile_stage_bytes(item_cols, G));
        const bool narrow_class = (p.flags & kFlagNoNarrowClass) == 0u;
        const int class_of_cols = item_cols;
        const uint32_t class_bytes =
            static_cast<uint32_t>(tile_stage_bytes(stage_class_cols(class_of_cols, narrow_class), G));
        if (class_bytes != stage_bytes) {
          // Another stage geometry: wait until every stage of the old ring has been
          // consumed (the new stages overlap them), then start over at stage 0.
          for (int s = 0; s < num_stages && ok; ++s) {
            if (!mbar_wait_bounded(empty_bar(s), empty_parity(s), abort_flag, timeout_ns)) {
              report_status(p, abort_flag, ST_PRODUCER_SLOT_TIMEOUT, static_cast<uint32_t>(item));
              ok = false;
            }
          }
          if (!ok) break;
          stage_bytes = class_bytes;
          num_stages = tile_stages(stage_class_cols(class_of_cols, narrow_class), G);
          stage = 0;
          in_flight = 0;
        }
        // Arm a stage for the bytes of one K step of this item (for a CTA pair
        // both CTAs' loads complete on the leader's barrier, armed for both).
        auto arm = [&](uint32_t s) {
          if constexpr (G == 1) {
            mbar_arrive_expect_tx(full_bar(s), item_bytes);
          } else {
            if (cta_rank == 0) mbar_arrive_expect_tx(full_bar(s), 2 * item_bytes);
          }
          fills ^= 1u << s;
        };
        // A carries no L2 hint: its rows are read by the items of one M tile and then
        // dead, while W (evict-last) is read again by every round of items.
        auto load_a = [&](uint32_t s, int kt) {
          const uint32_t dst = smem_base + s * stage_bytes;
          const uint32_t bar = (G == 2) ? leader_full0 + 8u * s : full_bar(s);
          if constexpr (G == 1) {
            tma_load_2d(dst, &p.map_a, kt * kBlockK, a_row0, bar);
          } else {
            tma_load_2d_pair(dst, &p.map_a, kt * kBlockK, a_row0, bar);
          }
        };
        // W boxes of the item's one or two parts: tensor map, first row and offset inside a stage.
        const int rows0 = tile_b_rows(w.part_cols[0], G);
        const CUtensorMap* const map0 = &p.map_b[w.part_cols[0] / kUnit - 1];
        const int w_row0 = w.n0 + static_cast<int>(cta_rank) * rows0;
        const bool two_parts = kAllowWide && (w.parts == 2);
        const int rows1 = two_parts ? tile_b_rows(w.part_cols[1], G) : 0;
        const CUtensorMap* const map1 = &p.map_b[two_parts ? w.part_cols[1] / kUnit - 1 : 0];
        const int w_row1 = w.n0 + w.part_cols[0] + static_cast<int>(cta_rank) * rows1;
        const uint32_t w_off1 = Cfg::kABytes + static_cast<uint32_t>(rows0) * kBlockK * 2;
        auto load_box = [&](uint32_t dst, const CUtensorMap* map, int kt, int row0, uint32_t bar) {
          if constexpr (G == 1) {
            if (hints) tma_load_2d_hint(dst, map, kt * kBlockK, row0, bar, keep);
            else tma_load_2d(dst, map, kt * kBlockK, row0, bar);
          } else {
            if (hints) tma_load_2d_pair_hint(dst, map, kt * kBlockK, row0, bar, keep);
            else tma_load_2d_pair(dst, map, kt * kBlockK, row0, bar);
          }
        };
        auto load_w = [&](uint32_t s, int kt) {
          const uint32_t base = smem_base + s * stage_bytes;
          const uint32_t bar = (G == 2) ? leader_full0 + 8u * s : full_bar(s);
          load_box(base + Cfg::kABytes, map0, kt, w_row0, bar);
          if (two_parts) load_box(base + w_off1, map1, kt, w_row1, bar);
        };
        int kt_begin = 0;
        if constexpr (MODE == MODE_PULL) {
          // Gate on the pull workers having finished this 128-row panel.
          const int groups_per_panel = kBlockM / p.pull_rows;
          const int groups_total = (p.M + p.pull_rows - 1) / p.pull_rows;
          int groups = groups_total - panel * groups_per_panel;
          groups = groups < 0 ? 0 : (groups > groups_per_panel ? groups_per_panel : groups);
          const unsigned long long want = p.epoch1 * static_cast<unsigned long long>(groups) *
                                          static_cast<unsigned long long>(p.up) * static_cast<unsigned long long>(p.pull_segs);
          const uint64_t* ready = reinterpret_cast<const uint64_t*>(p.ready + panel);
          if (groups > 0 && ld_acquire_gpu_u64(ready) < want) {
            // The panel is still being pulled. W does not depend on it: arm the
            // stages that are free right now and load their W boxes, so that only
            // the A boxes remain to be fetched once the gate opens.
            int pre = 0;
            if ((p.flags & kFlagNoWPrefetch) == 0u) {
              uint32_t s = stage;
              while (pre < num_stages && pre < p.k_tiles && mbar_test_wait(empty_bar(s), empty_parity(s))) {
                arm(s);
                load_w(s, pre);
                advance(s);
                ++pre;
              }
            }
            const uint64_t t0 = globaltimer_ns();
            const long long gate_c0 = trace ? clock64() : 0;
            uint32_t it = 0;
            while (ld_acquire_gpu_u64(ready) < want) {
              if ((++it & 0x3fu) == 0) {
                if (*abort_flag != 0u || globaltimer_ns() - t0 > timeout_ns) {
                  report_status(p, abort_flag, ST_PULL_READY_TIMEOUT, static_cast<uint32_t>(panel));
                  ok = false;
                  break;
                }
                __nanosleep(64);
              }
            }
            if (trace) trace[kTraceGateCycles] += static_cast<unsigned long long>(clock64() - gate_c0);
            if (ok) fence_proxy_async_all();  // generic-proxy writes of dy -> async-proxy (TMA) reads
            // Armed stages get their A boxes even when giving up (with the gate
            // closed the rows are stale, never out of bounds), so that every armed
            // barrier completes and the drain below can count on it.
            for (int j = 0; j < pre; ++j) {
              load_a(stage, j);
              if (in_flight < static_cast<uint32_t>(num_stages)) ++in_flight;
              advance(stage);
            }
            kt_begin = pre;
            if (!ok) break;
          } else if (groups > 0) {
            fence_proxy_async_all();
          }
          if (trace && trace[kTraceGateFirstNs] == 0) trace[kTraceGateFirstNs] = globaltimer_ns() - trace[kTraceNsStart];
        }
        for (int kt = kt_begin; kt < p.k_tiles; ++kt) {
          const long long t_wait = trace ? clock64() : 0;
          const bool free_stage = mbar_wait_bounded(empty_bar(stage), empty_parity(stage), abort_flag, timeout_ns,
                                                    (p.flags & kFlagSpinWaits) != 0u);
          if (trace) waited += clock64() - t_wait;
          if (!free_stage) {
            report_status(p, abort_flag, ST_PRODUCER_SLOT_TIMEOUT, static_cast<uint32_t>(item));
            ok = false;
            break;
          }
          // Stage layout: [A box][W box of part 0][W box of part 1], every box 64 K elements wide.
          arm(stage);
          load_a(stage, kt);
          load_w(stage, kt);
          if (in_flight < static_cast<uint32_t>(num_stages)) ++in_flight;
          advance(stage);
        }
      }
      if (trace) trace[kTraceProdWait] = static_cast<unsigned long long>(waited);
      if (!ok) {
        // Giving up: let loads that are still in flight land before the CTA
        // retires. A lone CTA (and the leader of a pair) watches its own full
        // barriers (the phase of a stage's latest arming has the parity of
        // uses - 1); the other CTA of a pair has no barrier of its own to watch
        // and allows the same time.
        uint32_t s = stage;
        for (uint32_t i = 0; i < in_flight; ++i) {
          if (s == 0) s = static_cast<uint32_t>(num_stages);
          --s;
          const uint64_t t0 = globaltimer_ns();
          if (G == 1 || cta_rank == 0) {
            while (!mbar_try_wait(full_bar(s), ((fills >> s) & 1u) ^ 1u) && globaltimer_ns() - t0 < 2000000ull) {
            }
          } else {
            while (globaltimer_ns() - t0 < 2000000ull / static_cast<uint64_t>(num_stages > 0 ? num_stages : 1)) {
            }
          }
        }
      }
    }
  }

  // --------------------------------------------------------------- MMA issue
  // The whole warp runs this loop in lock-step and one elected lane issues the
  // tcgen05 instructions. Measured in isolation on resident operands (SM cycles
  // per 64-wide K step, 512 of them tensor-pipe work at N = 256): ~770 for a loop
  // run by a single lane inside a divergent branch, ~560 for the warp-uniform
  // loop with poll, four MMAs and commit as separate statements, 512 for the
  // fused sequence used here (umma_kstep4_probe_next / umma_kstep8_probe_next),
  // which also keeps the pipe full at N = 128. Every K step of an item goes
  // through the fused sequence (separate statements for its first and last step
  // measured 3800 cycles, a whole pipeline refill, per item boundary), except
  // the skewed first and last steps of an item of two accumulators.
  if (warp == 1 && !misaligned && cta_rank == 0) {
    const uint64_t desc0 = make_kmajor_sw128_desc(smem_base);
    const bool pair_commit = (G == 2) && (p.flags & kFlagSplitCommit) == 0u;
    // The fused step needs, for a CTA pair, the commit that reaches both CTAs' barriers at once.
    const bool fused_ok = (G == 1 || pair_commit) && (p.flags & kFlagSeparateIssue) == 0u;
    auto commit_to = [&](uint32_t bar) {
      if constexpr (G == 1) {
        umma_commit_1(bar);
      } else {
        if (pair_commit) {
          umma_commit_2_mask(bar, 3);
        } else {
          umma_commit_2(mapa_cluster(bar, 0));
          umma_commit_2(mapa_cluster(bar, 1));
        }
      }
    };
    uint32_t stage = 0;
    uint32_t uses = 0;        // bit s: parity of the number of times stage s has been consumed
    int num_stages = 0;       // current ring (see the producer): length and stage size
    uint32_t stage_bytes = 0;
    uint32_t acc_it = 0;  // parts issued so far: part i uses accumulator slot i & 1
    bool failed = false;
    bool stage_ready = false;  // the probe of the previous step found this stage full
    bool first_mma = true;
    long long wait_full = 0, wait_acc = 0;
    int items_run = 0;
    uint32_t ahead = first_entry;
    for (int ordinal = 0, item = cluster_id;; ++ordinal, item += num_clusters, ++items_run) {
      uint32_t entry;
      const int got = next_item(ordinal, item, ahead, &entry);
      if (got < 0) {
        if (lane == 0) report_status(p, abort_flag, ST_ITEM_FEED_TIMEOUT, static_cast<uint32_t>(ordinal));
        failed = true;
      }
      if (got <= 0) break;
      const WorkItem w = decode_entry(entry);
      if (w.parts == 0) continue;
      {
        const int class_cols =
            stage_class_cols(w.part_cols[0] + w.part_cols[1], (p.flags & kFlagNoNarrowClass) == 0u);
        const uint32_t class_bytes = static_cast<uint32_t>(tile_stage_bytes(class_cols, G));
        if (class_bytes != stage_bytes) {
          // another stage geometry: everything issued so far has been consumed here,
          // the producer restarts at stage 0 as well
          stage_bytes = class_bytes;
          num_stages = tile_stages(class_cols, G);
          stage = 0;
          stage_ready = false;
        }
      }
      const uint64_t desc_step = static_cast<uint64_t>(stage_bytes >> 4);
      const uint32_t slot0 = acc_it & 1u, slot1 = slot0 ^ 1u;
      const uint32_t d_tmem0 = tmem_base + slot0 * kBlockN, d_tmem1 = tmem_base + slot1 * kBlockN;
      const uint32_t idesc0 = make_idesc_bf16(Cfg::kUmmaM, w.part_cols[0]);
      const uint32_t idesc1 = make_idesc_bf16(Cfg::kUmmaM, w.parts == 2 ? w.part_cols[1] : kUnit);
      const uint64_t b_off0 = static_cast<uint64_t>(Cfg::kABytes >> 4);
      const uint64_t b_off1 =
          b_off0 + static_cast<uint64_t>((static_cast<uint32_t>(tile_b_rows(w.part_cols[0], G)) * kBlockK * 2) >> 4);
      uint64_t a_desc = desc0 + desc_step * stage;
      // Wait (unless the previous step's probe saw it) until the operands of `stage` have landed.
      auto wait_operands = [&]() {
        if (!stage_ready) {
          const long long t_full = trace ? clock64() : 0;
          if (!mbar_wait_bounded(full_bar(stage), (uses >> stage) & 1u, abort_flag, timeout_ns,
                                 (p.flags & kFlagSpinWaits) != 0u)) {
            report_status(p, abort_flag, ST_MMA_FULL_TIMEOUT, static_cast<uint32_t>(item));
            failed = true;
          }
          if (trace) wait_full += clock64() - t_full;
          tc_fence_after_sync();
        }
      };
      auto next_of = [&](uint32_t s) { return (s + 1u == static_cast<uint32_t>(num_stages)) ? 0u : s + 1u; };
      // First and last K step: separate statements. The first waits for each
      // accumulator slot just before the MMAs that overwrite it, the last
      // publishes each part's accumulator as soon as that part's MMAs are issued.
      auto edge_step = [&](bool first, bool last) {
        wait_operands();
        uses ^= 1u << stage;
        for (int part = 0; part < w.parts; ++part) {
          const uint32_t slot = part == 0 ? slot0 : slot1;
          if (first) {
            // This part overwrites its accumulator slot: the epilogue must have read the slot's previous part.
            const uint32_t aphase = ((acc_it + part) >> 1) & 1u;
            const long long t_acc = trace ? clock64() : 0;
            if (!mbar_wait_bounded(acc_empty_bar(slot), aphase ^ 1u, abort_flag, timeout_ns)) {
              report_status(p, abort_flag, ST_MMA_ACC_TIMEOUT, static_cast<uint32_t>(item));
              failed = true;
            }
            if (trace) wait_acc += clock64() - t_acc;
            tc_fence_after_sync();
          }
          if (elect_one_sync()) {
            // 16 BF16 = 32 bytes further along K inside the 128-byte swizzle row per MMA.
            const uint32_t d = part == 0 ? d_tmem0 : d_tmem1;
            const uint32_t idesc = part == 0 ? idesc0 : idesc1;
            const uint64_t b_desc = a_desc + (part == 0 ? b_off0 : b_off1);
            umma_bf16<G>(d, a_desc, b_desc, idesc, first ? 0u : 1u);
            umma_bf16<G>(d, a_desc + 2, b_desc + 2, idesc, 1u);
            umma_bf16<G>(d, a_desc + 4, b_desc + 4, idesc, 1u);
            umma_bf16<G>(d, a_desc + 6, b_desc + 6, idesc, 1u);
            if (last) commit_to(acc_full_bar(slot));  // publish the finished accumulator to the epilogue warps
          }
        }
        // Release the shared-memory stage once these MMAs have read it.
        if (elect_one_sync()) commit_to(empty_bar(stage));
        stage_ready = false;
        stage = next_of(stage);
        a_desc = stage == 0u ? desc0 : a_desc + desc_step;
      };
      // Four MMAs of one part on the stage whose A descriptor is `a`.
      auto part_step = [&](int part, uint64_t a, bool overwrite) {
        if (elect_one_sync()) {
          const uint32_t d = part == 0 ? d_tmem0 : d_tmem1;
          const uint32_t idesc = part == 0 ? idesc0 : idesc1;
          const uint64_t b_desc = a + (part == 0 ? b_off0 : b_off1);
          umma_bf16<G>(d, a, b_desc, idesc, overwrite ? 0u : 1u);
          umma_bf16<G>(d, a + 2, b_desc + 2, idesc, 1u);
          umma_bf16<G>(d, a + 4, b_desc + 4, idesc, 1u);
          umma_bf16<G>(d, a + 6, b_desc + 6, idesc, 1u);
        }
      };
      auto wait_slot = [&](int part) {
        const uint32_t slot = part == 0 ? slot0 : slot1;
        const uint32_t aphase = ((acc_it + part) >> 1) & 1u;
        const long long t_acc = trace ? clock64() : 0;
        if (!mbar_wait_bounded(acc_empty_bar(slot), aphase ^ 1u, abort_flag, timeout_ns)) {
          report_status(p, abort_flag, ST_MMA_ACC_TIMEOUT, static_cast<uint32_t>(item));
          failed = true;
        }
        if (trace) wait_acc += clock64() - t_acc;
        tc_fence_after_sync();
      };
      // An item of two accumulators owns all of TMEM, so its K loop cannot start
      // before the epilogue has read the previous item. To shorten that wait the
      // first part runs kSkew K steps ahead of the second at both ends of the
      // item: at the end its accumulator is complete (and being read out) while
      // the second part still has kSkew steps to go, and at the start the second
      // part's slot is only needed kSkew steps after the first's. In between
      // both parts consume the same stage. The stages of the skewed steps are
      // released by the second part, the later reader. Each part still sees K
      // in ascending order.
      constexpr int kSkew = 2;
      const int k_last = p.k_tiles - 1;
      const bool skewed = kAllowWide && w.parts == 2 && fused_ok && p.k_tiles >= 2 * kSkew + 2 && num_stages > kSkew &&
                          (p.flags & kFlagNoPartSkew) == 0u;
      int kt_from = 0, kt_to = p.k_tiles;  // K steps [kt_from, kt_to) run as fused sequences
      if (skewed) {
        uint32_t held_stage[kSkew];
        uint64_t held_desc[kSkew];
        for (int j = 0; j < kSkew; ++j) {  // first part, steps 0 .. kSkew-1
          wait_operands();
          stage_ready = false;
          if (j == 0) wait_slot(0);
          part_step(0, a_desc, j == 0);
          held_stage[j] = stage;
          held_desc[j] = a_desc;
          stage = next_of(stage);
          a_desc = stage == 0u ? desc0 : a_desc + desc_step;
        }
        for (int j = 0; j < kSkew; ++j) {  // second part catches up and releases the stages
          if (j == 0) wait_slot(1);
          part_step(1, held_desc[j], j == 0);
          if (elect_one_sync()) commit_to(empty_bar(held_stage[j]));
          uses ^= 1u << held_stage[j];
        }
        kt_from = kSkew;
        kt_to = p.k_tiles - kSkew;
      } else if (fused_ok) {
        // The epilogue must have read the previous contents of the slots this item overwrites.
        wait_slot(0);
        if (kAllowWide && w.parts == 2) wait_slot(1);
      }
      // The MMAs of a stage, the commit that frees it and a probe of the next
      // stage's barrier as one instruction sequence of the elected lane.
      if (fused_ok) {
        if (!kAllowWide || w.parts == 1) {
          for (int kt = kt_from; kt < kt_to; ++kt) {
            wait_operands();
            uses ^= 1u << stage;
            const uint32_t next_stage = next_of(stage);
            uint32_t probed = 0;
            if (elect_one_sync()) {
              probed = umma_kstep4_probe_next<G>(d_tmem0, a_desc, a_desc + b_off0, idesc0, kt > 0 ? 1u : 0u,
                                                 empty_bar(stage), full_bar(next_stage), (uses >> next_stage) & 1u);
            }
            stage_ready = __any_sync(0xffffffffu, probed != 0u);
            stage = next_stage;
            a_desc = stage == 0u ? desc0 : a_desc + desc_step;
          }
        } else {
          for (int kt = kt_from; kt < kt_to; ++kt) {
            wait_operands();
            uses ^= 1u << stage;
            const uint32_t next_stage = next_of(stage);
            uint32_t probed = 0;
            if (elect_one_sync()) {
              probed = umma_kstep8_probe_next<G>(d_tmem0, d_tmem1, a_desc, a_desc + b_off0, a_desc + b_off1, idesc0,
                                                 idesc1, kt > 0 ? 1u : 0u, empty_bar(stage), full_bar(next_stage),
                                                 (uses >> next_stage) & 1u);
            }
            stage_ready = __any_sync(0xffffffffu, probed != 0u);
            stage = next_stage;
            a_desc = stage == 0u ? desc0 : a_desc + desc_step;
          }
        }
      } else {
        for (int kt = 0; kt < p.k_tiles; ++kt) edge_step(kt == 0, kt == k_last);
      }
      if (trace && first_mma && lane == 0) trace[kTraceFirstMmaNs] = globaltimer_ns() - trace[kTraceNsStart];
      first_mma = false;
      if (skewed) {
        uint32_t held_stage[kSkew];
        uint64_t held_desc[kSkew];
        for (int j = 0; j < kSkew; ++j) {  // first part, last kSkew steps
          wait_operands();
          stage_ready = false;
          part_step(0, a_desc, false);
          held_stage[j] = stage;
          held_desc[j] = a_desc;
          stage = next_of(stage);
          a_desc = stage == 0u ? desc0 : a_desc + desc_step;
        }
        if (elect_one_sync()) commit_to(acc_full_bar(slot0));  // first accumulator complete: the epilogue starts on it
        for (int j = 0; j < kSkew; ++j) {  // second part, last kSkew steps
          part_step(1, held_desc[j], false);
          if (elect_one_sync()) commit_to(empty_bar(held_stage[j]));
          uses ^= 1u << held_stage[j];
        }
        if (elect_one_sync()) commit_to(acc_full_bar(slot1));
      } else if (fused_ok) {
        // Publish the finished accumulators to the epilogue warps.
        if (elect_one_sync()) {
          commit_to(acc_full_bar(slot0));
          if (kAllowWide && w.parts == 2) commit_to(acc_full_bar(slot1));
        }
      }
      acc_it += static_cast<uint32_t>(kAllowWide ? w.parts : 1);
      // A lane whose wait ran out has raised the abort flag, which makes every
      // later wait return at once; the warp leaves together at an item boundary.
      if (__any_sync(0xffffffffu, failed)) break;
    }
    if (trace && lane == 0) {
      trace[kTraceMmaWaitFull] = static_cast<unsigned long long>(wait_full);
      trace[kTraceMmaWaitAcc] = static_cast<unsigned long long>(wait_acc);
      trace[kTraceItems] = static_cast<unsigned long long>(items_run);
    }
  }

  // ---------------------------------------------------------------- epilogue
  if (warp >= 2 && warp < 6 && !misaligned) {
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    uint8_t* epi_buf0 = smem + Cfg::kOffEpi + q * (kEpiBufs * kEpiBufBytes);
    float* bias_s = reinterpret_cast<float*>(smem + Cfg::kOffBias) + q * kEpiCols;
    const uint32_t acc_empty_leader0 =
        (G == 2) ? mapa_cluster(acc_empty_bar(0), 0) : acc_empty_bar(0);
    uint32_t acc_it = 0;
    uint32_t store_it = 0;
    bool ok = true;
    long long epi_wait = 0;
    bool handoff_checked = false;
    uint32_t ahead = first_entry;
    for (int ordinal = 0, item = cluster_id; ok; ++ordinal, item += num_clusters) {
      uint32_t entry;
      const int got = next_item(ordinal, item, ahead, &entry);
      if (got < 0) {
        if (lane == 0) report_status(p, abort_flag, ST_ITEM_FEED_TIMEOUT, static_cast<uint32_t>(ordinal));
        ok = false;
      }
      if (got <= 0) break;
      const WorkItem w = decode_entry(entry);
      if (w.parts == 0) continue;
      const int row0 = (w.m_idx * G + static_cast<int>(cta_rank)) * kBlockM + q * kEpiRows;
      int part_col0 = w.n0;
      for (int part = 0; part < (kAllowWide ? w.parts : 1) && ok; ++part, ++acc_it) {
        const uint32_t as = acc_it & 1u;
        const uint32_t aphase = (acc_it >> 1) & 1u;
        // The bias of a 64-column sub-tile is fetched one sub-tile ahead (here: before the
        // wait for the accumulator), so that its global-memory latency never sits
        // between two reads of TMEM: the slot is handed back after the last read.
        uint32_t bias_next = 0u;
        if (p.bias != nullptr && part_col0 < p.N)
          bias_next = *reinterpret_cast<const uint32_t*>(p.bias + part_col0 + 2 * lane);

        const long long t_epi = trace ? clock64() : 0;
        const bool got = mbar_wait_bounded(acc_full_bar(as), aphase, abort_flag, timeout_ns);
        if (trace) epi_wait += clock64() - t_epi;
        if (!__all_sync(0xffffffffu, got)) {
          if (lane == 0) report_status(p, abort_flag, ST_EPILOGUE_TIMEOUT, static_cast<uint32_t>(item));
          ok = false;
          break;
        }
        tc_fence_after_sync();

        const int chunks = w.part_cols[part] / kEpiCols;
        for (int c = 0; c < chunks; ++c) {
          const int gcol = part_col0 + c * kEpiCols;
          const bool in_range = gcol < p.N;
          // Bias for these 64 columns, widened to FP32, shared inside the warp.
          if (p.bias != nullptr) {
            const __nv_bfloat162 b2 = *reinterpret_cast<const __nv_bfloat162*>(&bias_next);
            bias_s[2 * lane] = __bfloat162float(b2.x);
            bias_s[2 * lane + 1] = __bfloat162float(b2.y);
            if (c + 1 < chunks && gcol + kEpiCols < p.N)
              bias_next = *reinterpret_cast<const uint32_t*>(p.bias + gcol + kEpiCols + 2 * lane);
          }
          uint32_t v[2][32];
          const uint32_t taddr =
              tmem_base + (static_cast<uint32_t>(q * 32) << 16) + as * kBlockN + c * kEpiCols;
          tmem_ld_32x32(taddr, v[0]);
          tmem_ld_32x32(taddr + 32, v[1]);
          tmem_ld_wait();
          if (c == chunks - 1) {
            // Accumulator fully read: hand the TMEM slot back to the MMA warp.
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
              if constexpr (G == 1) {
                mbar_arrive(acc_empty_bar(as));
              } else {
                mbar_arrive_cluster(acc_empty_leader0 + 8u * as);
              }
            }
          }
          __syncwarp();  // bias_s visible to the whole warp

          uint32_t packed[32];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              float lo = __uint_as_float(v[h][j]);
              float hi = __uint_as_float(v[h][j + 1]);
              if (p.bias != nullptr) {
                lo += bias_s[h * 32 + j];
                hi += bias_s[h * 32 + j + 1];
              }
              const __nv_bfloat162 r = __floats2bfloat162_rn(lo, hi);
              packed[h * 16 + j / 2] = *reinterpret_cast<const uint32_t*>(&r);
            }
          }

          // Staging buffer reuse: the store issued two sub-tiles ago must have
          // finished reading shared memory.
          if (lane == 0) bulk_wait_group_read<kEpiBufs - 1>();
          __syncwarp();
          uint8_t* buf = epi_buf0 + (store_it & 1u) * kEpiBufBytes;
          // Row `lane` = 128 bytes = 8 chunks of 16 bytes, chunk j stored at
          // position j ^ (lane & 7): the 128-byte swizzle the store map expects.
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint4 val = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2],
                                         packed[4 * j + 3]);
            *reinterpret_cast<uint4*>(buf + lane * 128 + ((j ^ (lane & 7)) << 4)) = val;
          }
          fence_proxy_async_smem();
          __syncwarp();
          if constexpr (MODE == MODE_PEER_WRITE) {
            // The slots may still be read by their owners (copy-out of the previous
            // operation): the first store of this warp waits for their hand-off.
            if (!handoff_checked) {
              handoff_checked = true;
              const bool handed = sync_wait_warp(p.sync, lane);
              if (lane == 0) {
                fence_proxy_async_all();  // the acquires above before the async-proxy stores below
                if (!handed) *abort_flag = 1u;
              }
              __syncwarp();
              if (!handed) {
                ok = false;
                break;
              }
            }
          }
          if (lane == 0) {
            if (row0 < p.M && in_range) {
              if constexpr (MODE == MODE_PEER_WRITE) {
                const int dst = gcol / p.shard;
                const int lcol = gcol - dst * p.shard;
                if ((p.flags & kFlagNoL2Hints) == 0u) {
                  tma_store_2d_hint(&p.map_out[dst], lcol, row0, smem_u32(buf), l2_policy_evict_first());
                } else {
                  tma_store_2d(&p.map_out[dst], lcol, row0, smem_u32(buf));
                }
              } else {
                if ((p.flags & kFlagNoL2Hints) == 0u) {
                  tma_store_2d_hint(&p.map_out[0], gcol, row0, smem_u32(buf), l2_policy_evict_first());
                } else {
                  tma_store_2d(&p.map_out[0], gcol, row0, smem_u32(buf));
                }
              }
            }
            bulk_commit_group();
          }
          ++store_it;
          __syncwarp();
        }
        part_col0 += w.part_cols[part];
      }
    }
    // Stores must have completed (not merely been read out of shared memory)
    // before the kernel ends and the hand-off flag is raised.
    if (lane == 0) bulk_wait_group<0>();
    __syncwarp();
    if (trace && warp == 2 && lane == 0) trace[kTraceEpiWait] = static_cast<unsigned long long>(epi_wait);
  }

  // ------------------------------------------------------------ pull workers
  // A ticket is one batch: up to 512 sixteen-byte vectors (pull_rows rows of one
  // peer shard), all loaded before the first is stored, so it costs one round
  // trip over NVLink. Tickets are numbered in the order the GEMM consumes
  // panels. One atomic draws a chunk of kPullChunk tickets (same-address atomics
  // serialise at ~8 ns each across the GPU, so one draw per ticket would be the
  // bottleneck); the chunk's tickets are `pull_stride` apart (the number of pull
  // warps in the grid), so that in their i-th round trip all warps together copy
  // the i-th run of consecutive tickets and panels complete in consumption
  // order. A ticket is published (proxy fence + release) while the next
  // ticket's loads are in flight.
  // Measured and rejected: letting the idle epilogue warps copy tickets during
  // start-up. More tickets in flight delayed the first panels (first gate open
  // after 23 us instead of 17 us on two GPUs), and a second inlined copy of the
  // ticket code in the kernel made this loop compile to something 1.7x slower
  // per ticket even when the copy never ran; keep the ticket code in one place.
  if constexpr (MODE == MODE_PULL) {
    if (warp >= 6 && !misaligned) {
      const unsigned long long total = static_cast<unsigned long long>(p.total_tickets);
      const unsigned long long stride = static_cast<unsigned long long>(p.pull_stride);
      const unsigned long long block = stride * kPullChunk;  // tickets covered by `stride` chunks
      const unsigned long long chunks = (total + block - 1) / block * stride;
      auto publish = [&](int panel) { pull_ticket_publish(p, panel, lane); };
      // The peers' staged shards are handed off by the tail of their staging copy.
      {
        const bool handed = sync_wait_warp(p.sync, lane);
        if (!handed && lane == 0) *abort_flag = 1u;
        __syncwarp();
      }
      // Every pull warp of the grid would issue its first ticket in the same
      // microsecond, and the link would deliver that first wave (7 MB) in no
      // particular order, all of it at about the same time. Pacing the first
      // tickets at about the rate the link delivers them makes them arrive in
      // ticket order, so the first panels complete first.
      if (p.pull_pace_ns != 0u) {
        const unsigned long long until =
            globaltimer_ns() + (static_cast<unsigned long long>(blockIdx.x) * kPullWarps + (warp - 6)) * p.pull_pace_ns;
        while (globaltimer_ns() < until) {
        }
      }
      int pending_panel = -1;
      int tickets_done = 0;
      const int lane_row0 = lane / (p.shard >> 3);  // lane's first vector inside a ticket
      const int lane_vec0 = lane - lane_row0 * (p.shard >> 3);
      // The first chunk of every pull warp is its own index (no cursor draw on the
      // critical path of the first panels); the cursor hands out the rest. Once
      // the cursor has run out, a warp looks for first chunks whose owner has
      // not shown up (a CTA that could not become resident because another
      // kernel holds its SM) and copies them in its place, so the CTAs that do
      // run never wait on one that does not.
      const unsigned long long me = static_cast<unsigned long long>(blockIdx.x) * kPullWarps + (warp - 6);
      unsigned long long c = me;
      bool copy_it = __shfl_sync(0xffffffffu, own_first_chunk ? 1 : 0, 0) != 0;
      bool stealing = false;
      unsigned long long steal_pos = 0;
      while (*abort_flag == 0u) {
        // Draw the next chunk now but read the result only after this chunk: at
        // kernel start every pull warp of the grid hits the cursor at once and the
        // same-address atomics take ~8 ns each, up to 7 us for the last warp.
        unsigned long long drawn = 0;
        if (!stealing && lane == 0) drawn = atomicAdd(p.cursor, 1ull);
        if (copy_it) {
          const unsigned long long t_first = (c / stride) * block + (c % stride);
          for (int i = 0; i < kPullChunk; ++i) {
            const unsigned long long t = t_first + static_cast<unsigned long long>(i) * stride;
            if (t >= total) break;
            const PullTicket k = pull_ticket_geometry(p, static_cast<uint32_t>(t));
            const int panel = k.panel;
            uint4 regs[kPullUnroll];
            pull_ticket_load(k, lane, regs);
            if (pending_panel >= 0) publish(pending_panel);
            pull_ticket_store(p, k, lane, lane_row0, lane_vec0, regs);
            __syncwarp();
            pending_panel = panel;
            if (tickets_done < 2) {
              // start-up: the first panels gate every CTA, publish them at once
              publish(pending_panel);
              pending_panel = -1;
              if (trace && tickets_done == 0 && warp == 6 && lane == 0)
                trace[kTracePullFirstNs] = globaltimer_ns() - trace[kTraceNsStart];
            }
            ++tickets_done;
          }
        }
        if (!stealing) {
          c = __shfl_sync(0xffffffffu, drawn, 0) - p.cursor_base + stride;
          copy_it = true;
          if (c >= chunks) {
            if (p.claimed == nullptr) break;
            stealing = true;
          }
        }
        if (stealing) {
          bool found = false;
          while (steal_pos < stride && !found) {
            const unsigned long long idx = steal_pos + static_cast<unsigned long long>(lane);
            const unsigned long long j = (me + 1ull + idx) % stride;
            const unsigned long long seen = (idx < stride) ? *reinterpret_cast<volatile unsigned long long*>(p.claimed + j)
                                                           : p.epoch1;
            uint32_t open = __ballot_sync(0xffffffffu, seen < p.epoch1);
            while (open != 0u && !found) {
              const int bit = __ffs(static_cast<int>(open)) - 1;
              open &= open - 1u;
              const unsigned long long jj = (me + 1ull + steal_pos + static_cast<unsigned long long>(bit)) % stride;
              unsigned long long before = p.epoch1;
              if (lane == 0) before = atomicMax(p.claimed + jj, p.epoch1);
              if (__shfl_sync(0xffffffffu, before < p.epoch1 ? 1 : 0, 0) != 0) {
                c = jj;
                found = true;
              }
            }
            if (open == 0u && !found) steal_pos += 32ull;
          }
          if (!found) break;
          copy_it = true;
        }
      }
      if (pending_panel >= 0) publish(pending_panel);
      // This warp will not read a peer arena again: once every pull warp of the
      // grid has said so, the peers may reuse their arenas.
      __syncwarp();
      if (lane == 0) sync_arrive_and_signal(p.sync);
      if (trace && lane == 0) {
        atomicMax(trace + kTracePullEndNs, static_cast<unsigned long long>(globaltimer_ns()));
        atomicAdd(trace + kTracePullTickets, static_cast<unsigned long long>(tickets_done));
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  __syncwarp();
  tc_fence_before_sync();
  if constexpr (G == 2) {
    __syncthreads();
    cluster_arrive_release();
    cluster_wait_acquire();
  } else {
    __syncthreads();
  }
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc<G>(tmem_base, kTmemCols);
  }
  if (fed && threadIdx.x == 0 && cta_rank == 0u) {
    // This CTA (pair) draws no more. The last one out leaves the feed as the
    // next launch expects it (a launch starts drawing only after the launch
    // before it has completed).
    if (atomicAdd(p.feed + 1, 1u) == static_cast<unsigned int>(num_clusters) - 1u) {
      p.feed[1] = 0u;
      p.feed[0] = 0u;
    }
  }
  if constexpr (MODE == MODE_PEER_WRITE) {
    // Every store of this CTA has completed (bulk wait in the epilogue warps,
    // then the barrier above): count the CTA in; the last one raises the flags.
    if (threadIdx.x == 0) {
      fence_proxy_async_global();
      sync_arrive_and_signal(p.sync);
    }
  }
  if (trace != nullptr && threadIdx.x == 0) {
    trace[kTraceEnd] = clock64();
    trace[kTraceNsEnd] = globaltimer_ns();
  }
}

}  // namespace mup
