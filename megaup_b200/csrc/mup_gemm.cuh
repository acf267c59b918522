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
// Tile: 128 (M) x 256 (N) x 64 (K) per CTA. G = 1 runs one CTA per tile
// (tcgen05 cta_group::1); G = 2 pairs two CTAs of a cluster on a 256x256
// tile (cta_group::2): each CTA loads its own 128 rows of A and its own 128
// rows of W, so no load is ever multicast.
//
// The FP32 accumulator of an output element is a single TMEM cell that
// receives the K products in ascending order, 16 at a time; bias is added in
// FP32 and the sum is rounded to BF16 once. Nothing about the schedule (tile
// width, which SM runs which tile, the half-width items of a partly filled
// last wave) changes that order, so every configuration gives the same bits.
//
// Schedule: persistent CTAs, static round-robin over work items in N-fastest
// order (peer-write: each rank starts at its own column block). The kernel
// is launched with programmatic stream serialization: it lets its successor
// be scheduled at entry and waits for its predecessor after its own set-up.
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
constexpr int kBlockN = 256;
constexpr int kBlockK = 64;           // K extent of one TMA box (128 bytes, the swizzle span)
#ifndef MUP_KSUB
#define MUP_KSUB 1
#endif
constexpr int kKSub = MUP_KSUB;              // boxes per pipeline stage (2 = 128-K stages with 8 MMAs per barrier round:
                                      // measured no faster, 3 deep stages hide less latency than 6 shallow ones)
constexpr int kStageK = kBlockK * kKSub;
constexpr int kUmmaK = 16;
constexpr int kMaxPeers = 8;
constexpr int kAccStages = 2;
constexpr int kTmemCols = 512;
constexpr int kEpiCols = 64;        // columns per epilogue sub-tile (128 bytes)
constexpr int kEpiRows = 32;        // rows per epilogue warp
constexpr int kEpiBufBytes = kEpiRows * kEpiCols * 2;  // 4096
constexpr int kEpiBufs = 2;
#ifndef MUP_PULL_MAX_VECS
#define MUP_PULL_MAX_VECS 512
#endif
constexpr int kPullMaxVecs = MUP_PULL_MAX_VECS;  // 16-byte vectors per pull ticket (one batch of peer loads per warp)
constexpr int kPullUnroll = kPullMaxVecs / 32;
constexpr int kPullWarps = 6;         // pull workers per CTA (warps 6 .. 6 + kPullWarps - 1)
constexpr int kPullChunk = 8;         // tickets drawn per atomic

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

// Shared-memory plan. The N width of a tile (`tile_n`: 128, 192 or 256) and with
// it the size and number of pipeline stages are chosen per problem on the
// host, so the layout keeps a fixed 192 KiB stage area and room for the
// largest stage count.
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
  static constexpr int kSmemBytes = kOffAbort + 4 + 56;         // small pad
  static constexpr int kUmmaM = kBlockM * G;
};

// W rows one CTA loads per stage, bytes of a stage, number of stages.
__host__ __device__ constexpr int tile_b_rows(int tile_n, int g) { return tile_n / g; }
__host__ __device__ constexpr int tile_stage_bytes(int tile_n, int g) {
  return kKSub * (kBlockM * kBlockK * 2 + tile_b_rows(tile_n, g) * kBlockK * 2);
}
__host__ __device__ constexpr int tile_stages(int tile_n, int g) {
  return kStageAreaBytes / tile_stage_bytes(tile_n, g) > kMaxStages
             ? kMaxStages
             : kStageAreaBytes / tile_stage_bytes(tile_n, g);
}

struct GemmParams {
  CUtensorMap map_a;                 // A  [M, K]   box 64 x 128
  CUtensorMap map_b;                 // W  [N, K]   box 64 x (tile_n/G)
  CUtensorMap map_b_half;            // W  [N, K]   box 64 x (tile_n/2G), for the split tail tiles
  CUtensorMap map_out[kMaxPeers];    // peer-write: [rows, shard] slot in peer p; pull: [0] = out [M, N]
  const __nv_bfloat16* bias;         // nullptr when absent
  uint32_t* status;                  // error word (host-visible)
  unsigned long long timeout_ns;
  int M, N, K;
  int shard;                         // exchanged columns per rank
  int up, rank;
  int n_rot;                         // peer-write: first N tile of this rank
  int m_tiles, n_tiles, k_tiles;     // m_tiles counts (128*G)-row tiles, n_tiles tile_n-column tiles
  int tile_n;                        // 128, 192 or 256 output columns per tile
  int split_tiles;                   // this many trailing tiles are each run as two half-width tiles (0: none)
  // pull mode only
  const __nv_bfloat16* peers[kMaxPeers];  // staged arenas [up(dest), peer_rows, shard]
  __nv_bfloat16* dy;                 // dense pulled input [M, K]
  unsigned long long* ready;         // [ceil(M/128)] monotonically increasing ticket counts
  unsigned long long* cursor;        // monotonically increasing cursor, in chunks of kPullChunk tickets
  unsigned long long epoch1;         // launch ordinal, 1-based
  unsigned long long cursor_base;    // cursor value that means "chunk 0" for this launch
  int peer_rows;
  int total_tickets;
  int pull_stride;                   // pull warps in the grid: distance between the tickets of a chunk
  int pull_rows;                     // rows per pull ticket: a power of two <= 16 with pull_rows * shard / 8 <= kPullMaxVecs
  int pull_segs;                     // column segments per shard row (> 1 only when one row exceeds a ticket; then pull_rows = 1)
  int pull_seg_vecs;                 // 16-byte vectors per segment
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
constexpr int kTraceSlots = 16;

constexpr unsigned int kFlagNoL2Hints = 8u;     // tuning: drop the L2 hints (W loads evict-last, output stores evict-first)
constexpr unsigned int kFlagSplitCommit = 1u;  // G=2: one commit per CTA of the pair instead of one for both
constexpr unsigned int kFlagSeparateIssue = 2u;  // tuning: poll, MMAs and commit as separate statements (the slower issue loop)
constexpr unsigned int kFlagPullExtraFence = 16u;  // tuning: an explicit fence.acq_rel.gpu before every release of a ready count

__device__ __forceinline__ void report_status(const GemmParams& p, volatile uint32_t* abort_flag,
                                              uint32_t code, uint32_t detail) {
  *abort_flag = 1u;
  if (p.status != nullptr) {
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

__device__ __forceinline__ PullTicket pull_ticket_geometry(const GemmParams& p, unsigned long long t) {
  const int vec_per_row = p.shard >> 3;
  const unsigned long long per_group = static_cast<unsigned long long>(p.up) * p.pull_segs;
  const int grp = static_cast<int>(t / per_group);
  const int within = static_cast<int>(t - static_cast<unsigned long long>(grp) * per_group);
  const int seg = within % p.pull_segs;
  int src_rank = within / p.pull_segs + p.rank + 1;
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
  k.panel = grp / (kBlockM / p.pull_rows);
  return k;
}

__device__ __forceinline__ void pull_ticket_load(const GemmParams& p, const PullTicket& k, int lane,
                                                 uint4 (&regs)[kPullUnroll]) {
  const int vec_per_row = p.shard >> 3;
#pragma unroll
  for (int u = 0; u < kPullUnroll; ++u) {
    const int vidx = u * 32 + lane;
    if (vidx < k.nvec) {
      const int rr = vidx / vec_per_row;
      const int cc = vidx - rr * vec_per_row;
      regs[u] = ld_stream_v4(k.src + static_cast<size_t>(rr) * p.shard + cc * 8);
    }
  }
}

__device__ __forceinline__ void pull_ticket_store(const GemmParams& p, const PullTicket& k, int lane,
                                                  const uint4 (&regs)[kPullUnroll]) {
  const int vec_per_row = p.shard >> 3;
#pragma unroll
  for (int u = 0; u < kPullUnroll; ++u) {
    const int vidx = u * 32 + lane;
    if (vidx < k.nvec) {
      const int rr = vidx / vec_per_row;
      const int cc = vidx - rr * vec_per_row;
      *reinterpret_cast<uint4*>(k.dst + static_cast<size_t>(rr) * p.K + cc * 8) = regs[u];
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

template <int G, int MODE>
__global__ void __launch_bounds__(kernel_threads(MODE), 1)
fused_exchange_gemm_kernel(const __grid_constant__ GemmParams p) {
  using Cfg = GemmCfg<G>;
  extern __shared__ __align__(1024) uint8_t smem[];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = (G == 2) ? cluster_ctarank() : 0u;
  const int cluster_id = blockIdx.x / G;
  const int num_clusters = gridDim.x / G;
  const int num_tiles = p.m_tiles * p.n_tiles;
  const int tile_n = p.tile_n;
  const int num_stages = tile_stages(tile_n, G);
  const uint32_t stage_bytes = static_cast<uint32_t>(tile_stage_bytes(tile_n, G));
  // Work items: the tiles of the full waves, then the tiles of the last,
  // partly filled wave cut into two half-width items each, so that the tail
  // keeps about twice as many SMs busy for half as long. An item keeps the
  // whole K loop of its columns, so the accumulation order is unchanged.
  const int split_from = num_tiles - p.split_tiles;
  const int num_items = num_tiles + p.split_tiles;
  auto decode_item = [&](int item, int& m_idx, int& n0, int& width) {
    int t = item;
    int half = 0;
    width = tile_n;
    if (item >= split_from) {
      const int j = item - split_from;
      t = split_from + (j >> 1);
      half = j & 1;
      width = tile_n >> 1;
    }
    m_idx = t / p.n_tiles;
    int n_blk = t - m_idx * p.n_tiles + p.n_rot;
    if (n_blk >= p.n_tiles) n_blk -= p.n_tiles;
    n0 = n_blk * tile_n + half * width;
  };

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

  // ------------------------------------------------------------------ set-up
  if (threadIdx.x == 0) {
    *abort_flag = 0u;
    if ((smem_base & 1023u) != 0u) report_status(p, abort_flag, ST_SMEM_MISALIGNED, smem_base);
    for (int s = 0; s < num_stages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < kAccStages; ++a) {
      mbar_init(acc_full_bar(a), 1);
      mbar_init(acc_empty_bar(a), 4 * G);
    }
    fence_mbar_init();
    tma_prefetch_desc(&p.map_a);
    tma_prefetch_desc(&p.map_b);
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
  // Everything above touched only this CTA's shared memory and TMEM; from here
  // on the kernel reads what earlier kernels of the stream wrote.
  grid_dep_wait();

  // ------------------------------------------------------------ TMA producer
  if (warp == 0 && !misaligned) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      uint32_t in_flight = 0;  // loads armed so far (saturates at kStages)
      bool ok = true;
      long long waited = 0;
      const uint32_t leader_full0 = (G == 2) ? mapa_cluster(full_bar(0), 0) : full_bar(0);
      const bool hints = (p.flags & kFlagNoL2Hints) == 0u;
      const uint64_t keep = l2_policy_evict_last();  // W is re-read by every wave of tiles
      for (int tile = cluster_id; tile < num_items && ok; tile += num_clusters) {
        int m_idx, n0, width;
        decode_item(tile, m_idx, n0, width);
        const int panel = m_idx * G + static_cast<int>(cta_rank);
        const int a_row0 = panel * kBlockM;
        const int b_rows = tile_b_rows(width, G);
        const int b_row0 = n0 + static_cast<int>(cta_rank) * b_rows;
        const CUtensorMap* map_b = (width == tile_n) ? &p.map_b : &p.map_b_half;
        const uint32_t item_bytes = static_cast<uint32_t>(tile_stage_bytes(width, G));
        if constexpr (MODE == MODE_PULL) {
          // Gate on the pull workers having finished this 128-row panel.
          const int groups_per_panel = kBlockM / p.pull_rows;
          const int groups_total = (p.M + p.pull_rows - 1) / p.pull_rows;
          int groups = groups_total - panel * groups_per_panel;
          groups = groups < 0 ? 0 : (groups > groups_per_panel ? groups_per_panel : groups);
          const unsigned long long want = p.epoch1 * static_cast<unsigned long long>(groups) *
                                          static_cast<unsigned long long>(p.up) * static_cast<unsigned long long>(p.pull_segs);
          if (groups > 0) {
            const uint64_t t0 = globaltimer_ns();
            const long long gate_c0 = trace ? clock64() : 0;
            uint32_t it = 0;
            while (ld_acquire_gpu_u64(reinterpret_cast<const uint64_t*>(p.ready + panel)) < want) {
              if ((++it & 0x3fu) == 0) {
                if (*abort_flag != 0u || globaltimer_ns() - t0 > timeout_ns) {
                  report_status(p, abort_flag, ST_PULL_READY_TIMEOUT, static_cast<uint32_t>(panel));
                  ok = false;
                  break;
                }
                __nanosleep(64);
              }
            }
            if (!ok) break;
            if (trace) {
              trace[kTraceGateCycles] += static_cast<unsigned long long>(clock64() - gate_c0);
              if (trace[kTraceGateFirstNs] == 0) trace[kTraceGateFirstNs] = globaltimer_ns() - trace[kTraceNsStart];
            }
            fence_proxy_async_all();  // generic-proxy writes of dy -> async-proxy (TMA) reads
          }
        }
        for (int kt = 0; kt < p.k_tiles; ++kt) {
          const long long t_wait = trace ? clock64() : 0;
          const bool free_stage = mbar_wait_bounded(empty_bar(stage), phase ^ 1u, abort_flag, timeout_ns);
          if (trace) waited += clock64() - t_wait;
          if (!free_stage) {
            report_status(p, abort_flag, ST_PRODUCER_SLOT_TIMEOUT, static_cast<uint32_t>(tile));
            ok = false;
            break;
          }
          // Stage layout: [A box 0][A box 1][B box 0][B box 1], every box 64 K elements wide.
          const uint32_t a_dst = smem_base + stage * stage_bytes;
          const uint32_t b_dst = a_dst + kKSub * Cfg::kABytes;
          const uint32_t b_box_bytes = static_cast<uint32_t>(b_rows) * kBlockK * 2;
          if constexpr (G == 1) {
            mbar_arrive_expect_tx(full_bar(stage), item_bytes);
#pragma unroll
            for (int sub = 0; sub < kKSub; ++sub) {
              const int kcol = kt * kStageK + sub * kBlockK;
              tma_load_2d(a_dst + sub * Cfg::kABytes, &p.map_a, kcol, a_row0, full_bar(stage));
              if (hints) {
                tma_load_2d_hint(b_dst + sub * b_box_bytes, map_b, kcol, b_row0, full_bar(stage), keep);
              } else {
                tma_load_2d(b_dst + sub * b_box_bytes, map_b, kcol, b_row0, full_bar(stage));
              }
            }
          } else {
            // Both CTAs' loads complete on the leader's barrier, which the
            // leader arms for the bytes of the whole pair.
            const uint32_t bar = leader_full0 + 8u * stage;
            if (cta_rank == 0) mbar_arrive_expect_tx(full_bar(stage), 2 * item_bytes);
#pragma unroll
            for (int sub = 0; sub < kKSub; ++sub) {
              const int kcol = kt * kStageK + sub * kBlockK;
              tma_load_2d_pair(a_dst + sub * Cfg::kABytes, &p.map_a, kcol, a_row0, bar);
              if (hints) {
                tma_load_2d_pair_hint(b_dst + sub * b_box_bytes, map_b, kcol, b_row0, bar, keep);
              } else {
                tma_load_2d_pair(b_dst + sub * b_box_bytes, map_b, kcol, b_row0, bar);
              }
            }
          }
          if (in_flight < static_cast<uint32_t>(num_stages)) ++in_flight;
          if (++stage == static_cast<uint32_t>(num_stages)) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (trace) trace[kTraceProdWait] = static_cast<unsigned long long>(waited);
      if (!ok && G == 1) {
        // Giving up: let loads that are still in flight land before the CTA
        // retires (their barrier completes without any consumer).
        uint32_t s = stage, ph = phase;
        for (uint32_t i = 0; i < in_flight; ++i) {
          if (s == 0) {
            s = static_cast<uint32_t>(num_stages);
            ph ^= 1u;
          }
          --s;
          const uint64_t t0 = globaltimer_ns();
          while (!mbar_try_wait(full_bar(s), ph) && globaltimer_ns() - t0 < 2000000ull) {
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
  // fused sequence used here (umma_kstep4_probe_next), which also keeps the pipe
  // full at N = 128. In the full kernel the last step makes no measurable
  // difference: the K loop is then limited by operand delivery from L2.
  if (warp == 1 && !misaligned && cta_rank == 0) {
    const uint32_t idesc_full = make_idesc_bf16(Cfg::kUmmaM, tile_n);
    const uint32_t idesc_half = make_idesc_bf16(Cfg::kUmmaM, tile_n >> 1);
    const uint64_t desc0 = make_kmajor_sw128_desc(smem_base);
    const uint64_t desc_step = static_cast<uint64_t>(stage_bytes >> 4);
    const bool pair_commit = (G == 2) && (p.flags & kFlagSplitCommit) == 0u;
    // The fused step needs one TMA box per stage and, for a CTA pair, the commit
    // that reaches both CTAs' barriers at once.
    const bool fused_step = (kKSub == 1) && (G == 1 || pair_commit) && (p.flags & kFlagSeparateIssue) == 0u;
    uint32_t stage = 0, phase = 0;
    uint32_t acc_it = 0;
    bool failed = false;
    bool stage_ready = false;  // the probe of the previous step found this stage full
    long long wait_full = 0, wait_acc = 0;
    for (int tile = cluster_id; tile < num_items; tile += num_clusters, ++acc_it) {
      const uint32_t as = acc_it & 1u;
      const uint32_t aphase = (acc_it >> 1) & 1u;
      const bool half_item = tile >= split_from;
      const uint32_t idesc = half_item ? idesc_half : idesc_full;
      const uint64_t b_box_step =
          static_cast<uint64_t>((tile_b_rows(half_item ? (tile_n >> 1) : tile_n, G) * kBlockK * 2) >> 4);
      const long long t_acc = trace ? clock64() : 0;
      if (!mbar_wait_bounded(acc_empty_bar(as), aphase ^ 1u, abort_flag, timeout_ns)) {
        report_status(p, abort_flag, ST_MMA_ACC_TIMEOUT, static_cast<uint32_t>(tile));
        failed = true;
      }
      if (trace) wait_acc += clock64() - t_acc;
      tc_fence_after_sync();
      const uint32_t d_tmem = tmem_base + as * kBlockN;
      for (int kt = 0; kt < p.k_tiles; ++kt) {
        if (!stage_ready) {
          const long long t_full = trace ? clock64() : 0;
          if (!mbar_wait_bounded(full_bar(stage), phase, abort_flag, timeout_ns)) {
            report_status(p, abort_flag, ST_MMA_FULL_TIMEOUT, static_cast<uint32_t>(tile));
            failed = true;
          }
          if (trace) wait_full += clock64() - t_full;
          tc_fence_after_sync();
        }
        const uint64_t a_desc = desc0 + desc_step * stage;
        const uint64_t b_desc = a_desc + static_cast<uint64_t>((kKSub * Cfg::kABytes) >> 4);
        uint32_t next_stage = stage + 1u, next_phase = phase;
        if (next_stage == static_cast<uint32_t>(num_stages)) {
          next_stage = 0;
          next_phase ^= 1u;
        }
        if (fused_step) {
          // Four MMAs, the commit that frees the stage and a probe of the next
          // stage's barrier as one instruction sequence of the elected lane.
          uint32_t probed = 0;
          if (elect_one_sync()) {
            probed = umma_kstep4_probe_next<G>(d_tmem, a_desc, b_desc, idesc, kt > 0 ? 1u : 0u, empty_bar(stage),
                                               full_bar(next_stage), next_phase);
          }
          stage_ready = __any_sync(0xffffffffu, probed != 0u);
        } else {
          if (elect_one_sync()) {
            // Per box: 16 BF16 = 32 bytes further along K inside the 128-byte swizzle row per MMA.
#pragma unroll
            for (int sub = 0; sub < kKSub; ++sub) {
              const uint64_t a_sub = a_desc + static_cast<uint64_t>(sub) * (Cfg::kABytes >> 4);
              const uint64_t b_sub = b_desc + static_cast<uint64_t>(sub) * b_box_step;
              umma_bf16<G>(d_tmem, a_sub, b_sub, idesc, (kt > 0 || sub > 0) ? 1u : 0u);
              umma_bf16<G>(d_tmem, a_sub + 2, b_sub + 2, idesc, 1u);
              umma_bf16<G>(d_tmem, a_sub + 4, b_sub + 4, idesc, 1u);
              umma_bf16<G>(d_tmem, a_sub + 6, b_sub + 6, idesc, 1u);
            }
            // Release the shared-memory slot once these MMAs have read it.
            if constexpr (G == 1) {
              umma_commit_1(empty_bar(stage));
            } else if (pair_commit) {
              umma_commit_2_mask(empty_bar(stage), 3);
            } else {
              umma_commit_2(mapa_cluster(empty_bar(stage), 0));
              umma_commit_2(mapa_cluster(empty_bar(stage), 1));
            }
          }
          stage_ready = false;
        }
        stage = next_stage;
        phase = next_phase;
      }
      // Publish the finished accumulator to the epilogue warps.
      if (elect_one_sync()) {
        if constexpr (G == 1) {
          umma_commit_1(acc_full_bar(as));
        } else if (pair_commit) {
          umma_commit_2_mask(acc_full_bar(as), 3);
        } else {
          umma_commit_2(mapa_cluster(acc_full_bar(as), 0));
          umma_commit_2(mapa_cluster(acc_full_bar(as), 1));
        }
      }
      // A lane whose wait ran out has raised the abort flag, which makes every
      // later wait return at once; the warp leaves together at a tile boundary.
      if (__any_sync(0xffffffffu, failed)) break;
    }
    if (trace && lane == 0) {
      trace[kTraceMmaWaitFull] = static_cast<unsigned long long>(wait_full);
      trace[kTraceMmaWaitAcc] = static_cast<unsigned long long>(wait_acc);
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
    for (int tile = cluster_id; tile < num_items && ok; tile += num_clusters, ++acc_it) {
      int m_idx, n0, width;
      decode_item(tile, m_idx, n0, width);
      const uint32_t as = acc_it & 1u;
      const uint32_t aphase = (acc_it >> 1) & 1u;
      const int row0 = (m_idx * G + static_cast<int>(cta_rank)) * kBlockM + q * kEpiRows;

      const long long t_epi = trace ? clock64() : 0;
      const bool got = mbar_wait_bounded(acc_full_bar(as), aphase, abort_flag, timeout_ns);
      if (trace) epi_wait += clock64() - t_epi;
      if (!__all_sync(0xffffffffu, got)) {
        if (lane == 0) report_status(p, abort_flag, ST_EPILOGUE_TIMEOUT, static_cast<uint32_t>(tile));
        ok = false;
        break;
      }
      tc_fence_after_sync();

      const int chunks = width / kEpiCols;
      for (int c = 0; c < chunks; ++c) {
        const int gcol = n0 + c * kEpiCols;
        const bool in_range = gcol < p.N;  // the last tile of a row may hang over N
        // Bias for these 64 columns, widened to FP32, shared inside the warp.
        if (p.bias != nullptr && in_range) {
          const __nv_bfloat162 b2 =
              *reinterpret_cast<const __nv_bfloat162*>(p.bias + gcol + 2 * lane);
          bias_s[2 * lane] = __bfloat162float(b2.x);
          bias_s[2 * lane + 1] = __bfloat162float(b2.y);
        }
        uint32_t v[2][32];
        const uint32_t taddr =
            tmem_base + (static_cast<uint32_t>(q * 32) << 16) + as * kBlockN + c * kEpiCols;
        tmem_ld_32x32(taddr, v[0]);
        tmem_ld_32x32(taddr + 32, v[1]);
        tmem_ld_wait();
        if (c == chunks - 1) {
          // Accumulator fully read: hand the TMEM stage back to the MMA warp.
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
      int pending_panel = -1;
      int tickets_done = 0;
      // The first chunk of every pull warp is its own index (no atomic on the
      // critical path of the first panels); the cursor hands out the rest.
      unsigned long long c = static_cast<unsigned long long>(blockIdx.x) * kPullWarps + (warp - 6);
      while (c < chunks && *abort_flag == 0u) {
        // Draw the next chunk now but read the result only after this chunk: at
        // kernel start every pull warp of the grid hits the cursor at once and the
        // same-address atomics take ~8 ns each, up to 7 us for the last warp.
        unsigned long long drawn = 0;
        if (lane == 0) drawn = atomicAdd(p.cursor, 1ull);
        const unsigned long long t_first = (c / stride) * block + (c % stride);
        for (int i = 0; i < kPullChunk; ++i) {
          const unsigned long long t = t_first + static_cast<unsigned long long>(i) * stride;
          if (t >= total) break;
          const PullTicket k = pull_ticket_geometry(p, t);
          const int panel = k.panel;
          uint4 regs[kPullUnroll];
          pull_ticket_load(p, k, lane, regs);
          if (pending_panel >= 0) publish(pending_panel);
          pull_ticket_store(p, k, lane, regs);
          __syncwarp();
          pending_panel = panel;
          if (tickets_done < 2) {
            // start-up: the first panels gate every CTA, publish them at once
            publish(pending_panel);
            pending_panel = -1;
          }
          ++tickets_done;
        }
        c = __shfl_sync(0xffffffffu, drawn, 0) - p.cursor_base + stride;
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
