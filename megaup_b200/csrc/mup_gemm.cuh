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
// FP32 and the sum is rounded to BF16 once.
//
// Warp roles (192 threads, 256 in pull mode):
//   warp 0      TMA producer (one elected lane)
//   warp 1      TMEM allocation + MMA issue (one elected lane, leader CTA)
//   warps 2-5   epilogue; warp w owns TMEM lanes 32*(w%4) .. +31
//   warps 6-7   (pull mode) peer -> dy copy workers
//
// Every wait is bounded. A role that gives up records a code in *status,
// raises the CTA's abort flag so the other roles give up too, and all roles
// meet at the final barrier where TMEM is released.
#pragma once

#include "mup_ptx.cuh"

namespace mup {

constexpr int kBlockM = 128;
constexpr int kBlockN = 256;
constexpr int kBlockK = 64;
constexpr int kUmmaK = 16;
constexpr int kMaxPeers = 8;
constexpr int kAccStages = 2;
constexpr int kTmemCols = 512;
constexpr int kEpiCols = 64;        // columns per epilogue sub-tile (128 bytes)
constexpr int kEpiRows = 32;        // rows per epilogue warp
constexpr int kEpiBufBytes = kEpiRows * kEpiCols * 2;  // 4096
constexpr int kEpiBufs = 2;
constexpr int kPullRowsPerTicket = 16;
constexpr int kPullUnroll = 8;

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

template <int G>
struct GemmCfg {
  static constexpr int kStages = (G == 1) ? 4 : 6;
  static constexpr int kABytes = kBlockM * kBlockK * 2;         // 16 KB
  static constexpr int kBRows = kBlockN / G;                    // W rows this CTA loads
  static constexpr int kBBytes = kBRows * kBlockK * 2;          // 32 / 16 KB
  static constexpr int kStageBytes = kABytes + kBBytes;         // 48 / 32 KB
  static constexpr int kOffEpi = kStages * kStageBytes;         // 196608
  static constexpr int kOffBias = kOffEpi + 4 * kEpiBufs * kEpiBufBytes;
  static constexpr int kOffBar = kOffBias + 4 * kEpiCols * 4;
  // full[kStages], empty[kStages], acc_full[2], acc_empty[2]
  static constexpr int kNumBars = 2 * kStages + 2 * kAccStages;
  static constexpr int kOffTmemSlot = kOffBar + kNumBars * 8;
  static constexpr int kOffAbort = kOffTmemSlot + 4;
  static constexpr int kSmemBytes = kOffAbort + 4 + 56;         // small pad
  static constexpr int kUmmaM = kBlockM * G;
};

struct GemmParams {
  CUtensorMap map_a;                 // A  [M, K]   box 64 x 128
  CUtensorMap map_b;                 // W  [N, K]   box 64 x (256/G)
  CUtensorMap map_out[kMaxPeers];    // peer-write: [rows, shard] slot in peer p; pull: [0] = out [M, N]
  const __nv_bfloat16* bias;         // nullptr when absent
  uint32_t* status;                  // error word (host-visible)
  unsigned long long timeout_ns;
  int M, N, K;
  int shard;                         // exchanged columns per rank
  int up, rank;
  int n_rot;                         // peer-write: first N tile of this rank
  int m_tiles, n_tiles, k_tiles;     // m_tiles counts (128*G)-row tiles
  // pull mode only
  const __nv_bfloat16* peers[kMaxPeers];  // staged arenas [up(dest), peer_rows, shard]
  __nv_bfloat16* dy;                 // dense pulled input [M, K]
  unsigned long long* ready;         // [ceil(M/128)] monotonically increasing ticket counts
  unsigned long long* cursor;        // monotonically increasing ticket cursor
  unsigned long long epoch1;         // launch ordinal, 1-based
  unsigned long long cursor_base;    // cursor value that means "ticket 0" for this launch
  int peer_rows;
  int total_tickets;
  unsigned int flags;                // tuning switches (kFlag*)
  unsigned long long* trace;         // optional [grid][8] cycle counters (nullptr: off)
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
constexpr int kTraceSlots = 8;

constexpr unsigned int kFlagPairCommit = 1u;  // G=2: one commit to both CTAs instead of one per CTA

__device__ __forceinline__ void report_status(const GemmParams& p, volatile uint32_t* abort_flag,
                                              uint32_t code, uint32_t detail) {
  *abort_flag = 1u;
  if (p.status != nullptr) {
    *reinterpret_cast<volatile uint32_t*>(p.status) = (code << 24) | (detail & 0xFFFFFFu);
  }
}

template <int G, int MODE>
__global__ void __launch_bounds__(MODE == MODE_PULL ? 256 : 192, 1)
fused_exchange_gemm_kernel(const __grid_constant__ GemmParams p) {
  using Cfg = GemmCfg<G>;
  extern __shared__ __align__(1024) uint8_t smem[];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = (G == 2) ? cluster_ctarank() : 0u;
  const int cluster_id = blockIdx.x / G;
  const int num_clusters = gridDim.x / G;
  const int num_tiles = p.m_tiles * p.n_tiles;

  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + Cfg::kOffBar;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (Cfg::kStages + s); };
  auto acc_full_bar = [&](int a) { return bar_base + 8u * (2 * Cfg::kStages + a); };
  auto acc_empty_bar = [&](int a) { return bar_base + 8u * (2 * Cfg::kStages + kAccStages + a); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + Cfg::kOffTmemSlot);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + Cfg::kOffAbort);
  const uint64_t timeout_ns = p.timeout_ns;
  unsigned long long* trace = (p.trace != nullptr) ? p.trace + static_cast<size_t>(blockIdx.x) * kTraceSlots : nullptr;
  if (trace != nullptr && threadIdx.x == 0) {
    trace[kTraceStart] = clock64();
    trace[kTraceNsStart] = globaltimer_ns();
  }

  // ------------------------------------------------------------------ set-up
  if (threadIdx.x == 0) {
    *abort_flag = 0u;
    if ((smem_base & 1023u) != 0u) report_status(p, abort_flag, ST_SMEM_MISALIGNED, smem_base);
    for (int s = 0; s < Cfg::kStages; ++s) {
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

  // ------------------------------------------------------------ TMA producer
  if (warp == 0 && !misaligned) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      uint32_t in_flight = 0;  // loads armed so far (saturates at kStages)
      bool ok = true;
      long long waited = 0;
      const uint32_t leader_full0 = (G == 2) ? mapa_cluster(full_bar(0), 0) : full_bar(0);
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
        const int m_idx = tile / p.n_tiles;
        const int n_idx = tile - m_idx * p.n_tiles;
        int n_blk = n_idx + p.n_rot;
        if (n_blk >= p.n_tiles) n_blk -= p.n_tiles;
        const int panel = m_idx * G + static_cast<int>(cta_rank);
        const int a_row0 = panel * kBlockM;
        const int b_row0 = n_blk * kBlockN + static_cast<int>(cta_rank) * Cfg::kBRows;
        if constexpr (MODE == MODE_PULL) {
          // Gate on the pull workers having finished this 128-row panel.
          const int groups_per_panel = kBlockM / kPullRowsPerTicket;
          const int groups_total = (p.M + kPullRowsPerTicket - 1) / kPullRowsPerTicket;
          int groups = groups_total - panel * groups_per_panel;
          groups = groups < 0 ? 0 : (groups > groups_per_panel ? groups_per_panel : groups);
          const unsigned long long want =
              p.epoch1 * static_cast<unsigned long long>(groups) * static_cast<unsigned long long>(p.up);
          if (groups > 0) {
            const uint64_t t0 = globaltimer_ns();
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
          const uint32_t a_dst = smem_base + stage * Cfg::kStageBytes;
          const uint32_t b_dst = a_dst + Cfg::kABytes;
          if constexpr (G == 1) {
            mbar_arrive_expect_tx(full_bar(stage), Cfg::kStageBytes);
            tma_load_2d(a_dst, &p.map_a, kt * kBlockK, a_row0, full_bar(stage));
            tma_load_2d(b_dst, &p.map_b, kt * kBlockK, b_row0, full_bar(stage));
          } else {
            // Both CTAs' loads complete on the leader's barrier, which the
            // leader arms for the bytes of the whole pair.
            const uint32_t bar = leader_full0 + 8u * stage;
            if (cta_rank == 0) mbar_arrive_expect_tx(full_bar(stage), 2 * Cfg::kStageBytes);
            tma_load_2d_pair(a_dst, &p.map_a, kt * kBlockK, a_row0, bar);
            tma_load_2d_pair(b_dst, &p.map_b, kt * kBlockK, b_row0, bar);
          }
          if (in_flight < static_cast<uint32_t>(Cfg::kStages)) ++in_flight;
          if (++stage == Cfg::kStages) {
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
            s = Cfg::kStages;
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
  if (warp == 1 && !misaligned && cta_rank == 0) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(Cfg::kUmmaM, kBlockN);
      uint32_t stage = 0, phase = 0;
      uint32_t acc_it = 0;
      bool ok = true;
      long long wait_full = 0, wait_acc = 0;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters, ++acc_it) {
        const uint32_t as = acc_it & 1u;
        const uint32_t aphase = (acc_it >> 1) & 1u;
        const long long t_acc = trace ? clock64() : 0;
        const bool acc_free = mbar_wait_bounded(acc_empty_bar(as), aphase ^ 1u, abort_flag, timeout_ns);
        if (trace) wait_acc += clock64() - t_acc;
        if (!acc_free) {
          report_status(p, abort_flag, ST_MMA_ACC_TIMEOUT, static_cast<uint32_t>(tile));
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + as * kBlockN;
        for (int kt = 0; kt < p.k_tiles; ++kt) {
          const long long t_full = trace ? clock64() : 0;
          const bool filled = mbar_wait_bounded(full_bar(stage), phase, abort_flag, timeout_ns);
          if (trace) wait_full += clock64() - t_full;
          if (!filled) {
            report_status(p, abort_flag, ST_MMA_FULL_TIMEOUT, static_cast<uint32_t>(tile));
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_base + stage * Cfg::kStageBytes;
          const uint64_t a_desc = make_kmajor_sw128_desc(a_addr);
          const uint64_t b_desc = make_kmajor_sw128_desc(a_addr + Cfg::kABytes);
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {
            // 16 BF16 = 32 bytes further along K inside the 128-byte swizzle row
            const uint64_t koff = static_cast<uint64_t>((k * kUmmaK * 2) >> 4);
            umma_bf16<G>(d_tmem, a_desc + koff, b_desc + koff, idesc,
                         (kt > 0 || k > 0) ? 1u : 0u);
          }
          // Release the shared-memory slot once these MMAs have read it.
          if constexpr (G == 1) {
            umma_commit_1(empty_bar(stage));
          } else if (p.flags & kFlagPairCommit) {
            umma_commit_2_mask(empty_bar(stage), 3);
          } else {
            umma_commit_2(mapa_cluster(empty_bar(stage), 0));
            umma_commit_2(mapa_cluster(empty_bar(stage), 1));
          }
          if (++stage == Cfg::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        // Publish the finished accumulator to the epilogue warps.
        if constexpr (G == 1) {
          umma_commit_1(acc_full_bar(as));
        } else if (p.flags & kFlagPairCommit) {
          umma_commit_2_mask(acc_full_bar(as), 3);
        } else {
          umma_commit_2(mapa_cluster(acc_full_bar(as), 0));
          umma_commit_2(mapa_cluster(acc_full_bar(as), 1));
        }
      }
      if (trace) {
        trace[kTraceMmaWaitFull] = static_cast<unsigned long long>(wait_full);
        trace[kTraceMmaWaitAcc] = static_cast<unsigned long long>(wait_acc);
      }
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
    for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters, ++acc_it) {
      const int m_idx = tile / p.n_tiles;
      const int n_idx = tile - m_idx * p.n_tiles;
      int n_blk = n_idx + p.n_rot;
      if (n_blk >= p.n_tiles) n_blk -= p.n_tiles;
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

#pragma unroll 1
      for (int c = 0; c < kBlockN / kEpiCols; ++c) {
        const int gcol = n_blk * kBlockN + c * kEpiCols;
        // Bias for these 64 columns, widened to FP32, shared inside the warp.
        if (p.bias != nullptr) {
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
        if (c == kBlockN / kEpiCols - 1) {
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
        if (lane == 0) {
          if (row0 < p.M) {
            if constexpr (MODE == MODE_PEER_WRITE) {
              const int dst = gcol / p.shard;
              const int lcol = gcol - dst * p.shard;
              tma_store_2d(&p.map_out[dst], lcol, row0, smem_u32(buf));
            } else {
              tma_store_2d(&p.map_out[0], gcol, row0, smem_u32(buf));
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
  if constexpr (MODE == MODE_PULL) {
    if (warp >= 6 && !misaligned) {
      const int vec_per_row = p.shard >> 3;  // 16-byte vectors per shard row
      const unsigned long long total = static_cast<unsigned long long>(p.total_tickets);
      for (;;) {
        unsigned long long t = 0;
        if (lane == 0) t = atomicAdd(p.cursor, 1ull) - p.cursor_base;
        t = __shfl_sync(0xffffffffu, t, 0);
        if (t >= total || *abort_flag != 0u) break;
        const int grp = static_cast<int>(t / static_cast<unsigned long long>(p.up));
        int src_rank = static_cast<int>(t - static_cast<unsigned long long>(grp) * p.up) + p.rank + 1;
        if (src_rank >= p.up) src_rank -= p.up;
        const int r0 = grp * kPullRowsPerTicket;
        int nrows = p.M - r0;
        nrows = nrows > kPullRowsPerTicket ? kPullRowsPerTicket : nrows;
        const int nvec = nrows * vec_per_row;
        const __nv_bfloat16* src =
            p.peers[src_rank] +
            (static_cast<size_t>(p.rank) * p.peer_rows + r0) * static_cast<size_t>(p.shard);
        __nv_bfloat16* dst = p.dy + static_cast<size_t>(r0) * p.K +
                             static_cast<size_t>(src_rank) * p.shard;
        for (int base = 0; base < nvec; base += 32 * kPullUnroll) {
          uint4 regs[kPullUnroll];
          int rr[kPullUnroll], cc[kPullUnroll];
#pragma unroll
          for (int u = 0; u < kPullUnroll; ++u) {
            const int vidx = base + u * 32 + lane;
            rr[u] = vidx / vec_per_row;
            cc[u] = vidx - rr[u] * vec_per_row;
            if (vidx < nvec) {
              regs[u] = ld_stream_v4(src + static_cast<size_t>(rr[u]) * p.shard + cc[u] * 8);
            }
          }
#pragma unroll
          for (int u = 0; u < kPullUnroll; ++u) {
            const int vidx = base + u * 32 + lane;
            if (vidx < nvec) {
              *reinterpret_cast<uint4*>(dst + static_cast<size_t>(rr[u]) * p.K + cc[u] * 8) = regs[u];
            }
          }
        }
        __syncwarp();
        if (lane == 0) {
          fence_proxy_async_all();
          __threadfence();
          red_release_gpu_add_u64(reinterpret_cast<uint64_t*>(p.ready + grp / (kBlockM / kPullRowsPerTicket)),
                                  1ull);
        }
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
  if (trace != nullptr && threadIdx.x == 0) {
    trace[kTraceEnd] = clock64();
    trace[kTraceNsEnd] = globaltimer_ns();
  }
}

}  // namespace mup
