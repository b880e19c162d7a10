// CTA-pair form of the persistent GEMM: a cluster of two CTAs computes one 256 x BN tile with
// tcgen05.mma.cta_group::2.  Each CTA stages its own 128 rows of A and its own half of the B tile,
// so the shared-memory traffic per flop drops by a third against the one-CTA kernel and the
// operand reads of the tensor cores no longer compete with a full B tile per CTA.
//
// Same schedule semantics as gemm_kernel (waves in order, consumer flags, grouped raster inside a
// wave, here over 256-row tiles).  With FUSED the kernel also has the comm warp (one per CTA) and
// the routed epilogue of gemm_kernel: each CTA of a pair routes, counts and reduces its own 128
// rows of the tile.  No TMA load carries a multicast qualifier; only tcgen05.commit signals both
// CTAs' barriers.
#pragma once
#include "gemm_sm100.cuh"

namespace syn {

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `addr` (a shared::cta address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(rank));
  return out;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// 2-D tiled load into this CTA's shared memory whose completion is counted on the barrier at
// cluster address `bar_cluster_addr` (the pair leader's barrier); no multicast.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_holder, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
               ::"r"(smem_u32(smem_holder)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f16_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the barrier at this shared-memory offset in both CTAs of the pair once all MMAs issued
// so far have completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"(mask)
      : "memory");
}

constexpr int GEMM2_BM = 256;

// Tail splitting.  When the tile count leaves a small remainder after the last full persistent
// round, the remaining `tiles` tiles are not given a round of their own (which would idle most of
// the GPU): each is cut along K into `slices` pieces, one per CTA pair.  A piece is written as an
// fp32 partial tile to its own place in a workspace; when all 2 * slices CTAs of a tile have
// arrived (they run at the same time, the grid being persistent), each of them sums a share of the
// tile's rows over the slices in a fixed order, converts to 16 bit and stores.
struct PairTail {
  int tiles;            // 0 = no splitting
  int slices;
  int first_tile;       // tile id of the first tail tile (= full rounds * pairs)
  float* ws;            // [tiles][slices][256][BN] fp32 partial tiles (contents need not be kept)
  unsigned int* count;  // [2 * tiles] arrivals / departures, zero between launches
};

// Work item n of this pair: full-round tiles first, then (at most) one K slice of a tail tile.
struct PairWork {
  int tile, kb0, kb1;
  bool is_slice;
};
__device__ __forceinline__ bool pair_work(const GemmParams& p, const PairTail& tail, int total, int pair_id, int num_pairs,
                                          int n, PairWork& w) {
  w.kb0 = 0;
  w.kb1 = p.k_blocks;
  w.is_slice = false;
  if (tail.tiles == 0) {
    w.tile = pair_id + n * num_pairs;
    return w.tile < total;
  }
  const int rounds = tail.first_tile / num_pairs;  // the host makes first_tile a whole number of rounds
  if (n < rounds) {
    w.tile = pair_id + n * num_pairs;
    return true;
  }
  if (n == rounds && pair_id < tail.tiles * tail.slices) {
    w.tile = tail.first_tile + pair_id / tail.slices;
    const int sl = pair_id % tail.slices;
    w.kb0 = static_cast<int>(static_cast<long>(p.k_blocks) * sl / tail.slices);
    w.kb1 = static_cast<int>(static_cast<long>(p.k_blocks) * (sl + 1) / tail.slices);
    w.is_slice = true;
    return w.kb1 > w.kb0;
  }
  return false;
}

// Tile cursor over 256-row tiles (two 128-row tile rows of the wave table per tile).
struct PairCursor {
  int wave = 0;
  int past = 0;
  __device__ __forceinline__ bool seek(const GemmParams& p, int tile, int& m2_blk, int& n_blk) {
    bool moved = false;
    while (true) {
      const int cnt = (p.waves[wave].tiles_m >> 1) * p.waves[wave].tiles_n;
      if (tile < past + cnt) break;
      past += cnt;
      ++wave;
      moved = true;
    }
    const int local = tile - past;
    const int tm = p.waves[wave].tiles_m >> 1, tn = p.waves[wave].tiles_n;
    const int in_group = p.group_m * tn;
    const int group_id = local / in_group;
    const int first_m = group_id * p.group_m;
    const int gsz = min(tm - first_m, p.group_m);
    const int r = local - group_id * in_group;
    m2_blk = first_m + (r % gsz) + (p.waves[wave].off_m >> 1);
    n_blk = (r / gsz) + p.waves[wave].off_n;
    return moved;
  }
};

template <int BN, int STAGES, bool FUSED>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm2_kernel(const __grid_constant__ GemmParams p, const __grid_constant__ CUtensorMap tmap_b_half,
             const int total_pair_tiles, const PairTail tail) {
  constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;         // this CTA's 128 rows of A
  constexpr int B_BYTES = (BN / 2) * GEMM_BK * 2;        // this CTA's half of the B tile
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_BYTES;
  uint8_t* ring = smem + STAGES * STAGE_BYTES;  // FUSED only: comm ring / epilogue staging
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring + (FUSED ? COMM_NBUF * COMM_PIECE : 0));
  uint64_t* full_bar = bars;                    // leader's copy counts both CTAs' bytes
  uint64_t* empty_bar = bars + STAGES;          // signalled in both CTAs by the leader's commits
  uint64_t* tfull_bar = bars + 2 * STAGES;      // [2], signalled in both CTAs
  uint64_t* tempty_bar = bars + 2 * STAGES + 2; // [2], leader's copy collects both CTAs' epilogue warps
  uint64_t* comm_bar = bars + 2 * STAGES + 4;   // [COMM_NBUF]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(comm_bar + COMM_NBUF);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_holder + 1);
  int* abort_info = const_cast<int*>(abort_word) + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();
  const bool leader = cta_rank == 0;
  const int pair_id = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  constexpr uint32_t TMEM_COLS = (2 * BN <= 256) ? 256 : 512;
  constexpr int ACC_STRIDE = TMEM_COLS / 2;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull_bar[i], 1);
      mbar_init(&tempty_bar[i], 8);  // four epilogue warps of each CTA
    }
    for (int i = 0; i < COMM_NBUF; ++i) mbar_init(&comm_bar[i], 1);
    *abort_word = 0;
    abort_info[0] = -1;
    abort_info[1] = -1;
    fence_mbar_init();
  }
  if (warp == 2) {
    tmem_alloc_pair(tmem_holder, TMEM_COLS);
    tmem_relinquish_pair();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tmap(&p.tmap_a);
    prefetch_tmap(&tmap_b_half);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  if (p.trace != nullptr && threadIdx.x == 0) atomicMin(&p.trace[0], globaltimer_ns());

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      PairCursor cur;
      int stage = 0;
      uint32_t phase = 0;
      uint32_t issued = 0;
      int gates_passed = 0;
      bool first = true;
      bool gave_up = false;
      PairWork wk;
      for (int n = 0; !gave_up && pair_work(p, tail, total_pair_tiles, pair_id, num_pairs, n, wk); ++n) {
        int m2_blk, n_blk;
        const bool moved = cur.seek(p, wk.tile, m2_blk, n_blk);
        if (moved || first) {
          const int sig = p.waves[cur.wave].csig;
          if (sig >= 0 && p.csig != nullptr) {
            const unsigned long long t_wait0 = p.trace != nullptr ? globaltimer_ns() : 0ull;
            if (!flag_wait_ge(p.csig + sig, p.signal_value, abort_word, p.timeout_ns)) {
              if (abort_info[0] < 0) {
                abort_info[0] = cur.wave;
                abort_info[1] = sig;
              }
              gave_up = true;  // the wave's data never arrived: issue no load for it
            }
            fence_proxy_async();
            if (p.trace != nullptr) {
              const unsigned long long t_wait1 = globaltimer_ns();
              atomicMin(&p.trace[2 + 3 * cur.wave], t_wait0);
              atomicMax(&p.trace[3 + 3 * cur.wave], t_wait1);
              atomicAdd(&p.trace[4 + 3 * cur.wave], t_wait1 - t_wait0);
            }
          }
          first = false;
        }
        const int row0 = m2_blk * GEMM2_BM + static_cast<int>(cta_rank) * GEMM_BM;
        const int col0 = n_blk * BN + static_cast<int>(cta_rank) * (BN / 2);
        // (K gates and K slices of tail tiles do not occur together: the host splits no tail then)
        const int ranges = p.num_kgates > 0 ? p.num_kgates : 1;
        for (int g = 0; g < ranges && !gave_up; ++g) {
          int kb_lo = wk.kb0, kb_hi = wk.kb1;
          if (p.num_kgates > 0) {
            kb_lo = p.kgate_kb0[g];
            kb_hi = p.kgate_kb1[g];
            if (g >= gates_passed) {
              if (p.kgate_sig[g] >= 0 && p.csig != nullptr &&
                  !flag_wait_ge(p.csig + p.kgate_sig[g], p.signal_value, abort_word, p.timeout_ns)) {
                if (abort_info[0] < 0) {
                  abort_info[0] = g;
                  abort_info[1] = p.kgate_sig[g];
                }
                gave_up = true;
                break;
              }
              fence_proxy_async();
              gates_passed = g + 1;
            }
          }
          for (int kb = kb_lo; kb < kb_hi; ++kb) {
            if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_word, p.timeout_ns)) {
              gave_up = true;
              break;
            }
            if (leader) mbar_expect_tx(&full_bar[stage], 2 * STAGE_BYTES);
            const uint32_t bar = map_to_cta(smem_u32(&full_bar[stage]), 0);
            tma_load_2d_pair(sA + stage * A_BYTES, &p.tmap_a, bar, kb * GEMM_BK, row0);
            tma_load_2d_pair(sB + stage * B_BYTES, &tmap_b_half, bar, kb * GEMM_BK, col0);
            ++issued;
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
      }
      if (*abort_word != 0 && leader) {
        // Loads already issued keep writing shared memory.  The leader's full barriers count both
        // CTAs' bytes, and the cluster barrier at the end keeps the other CTA alive meanwhile.
        for (int s = 0; s < STAGES; ++s)
          drain_stage(&full_bar[s], issued / STAGES + (static_cast<uint32_t>(s) < issued % STAGES ? 1u : 0u), p.timeout_ns);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (pair leader only)
    // The whole warp walks the work items and waits on the barriers; one elected lane issues each
    // tcgen05 instruction.
    if (leader) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      const uint32_t desc_hi = static_cast<uint32_t>(make_smem_desc_sw128(0, 16, 1024) >> 32);
      const uint32_t a_lo0 = static_cast<uint32_t>(make_smem_desc_sw128(smem_u32(sA), 16, 1024));
      const uint32_t b_lo0 = static_cast<uint32_t>(make_smem_desc_sw128(smem_u32(sB), 16, 1024));
      const uint32_t idesc = p.idesc;
      const uint64_t timeout_ns = p.timeout_ns;
      PairWork wk;
      for (int n = 0; pair_work(p, tail, total_pair_tiles, pair_id, num_pairs, n, wk); ++n) {
        if (*abort_word != 0) break;
        mbar_wait(&tempty_bar[acc], acc_phase ^ 1u, abort_word, timeout_ns);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * ACC_STRIDE);
        for (int kb = wk.kb0; kb < wk.kb1; ++kb) {
          mbar_wait(&full_bar[stage], phase, abort_word, timeout_ns);
          tc_fence_after();
          const uint32_t a_lo = a_lo0 + static_cast<uint32_t>(stage) * (A_BYTES >> 4);
          const uint32_t b_lo = b_lo0 + static_cast<uint32_t>(stage) * (B_BYTES >> 4);
#pragma unroll
          for (int k = 0; k < GEMM_BK / GEMM_UMMA_K; ++k) {
            if (elect_one())
              umma_ss_words_pair(d_tmem, a_lo + 2u * k, desc_hi, b_lo + 2u * k, desc_hi, idesc,
                                 ((kb - wk.kb0) | k) != 0 ? 1u : 0u);
          }
          if (elect_one()) umma_commit_pair(&empty_bar[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (elect_one()) umma_commit_pair(&tfull_bar[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else if (warp == 3) {
    // ------------------------------------------------------------ comm warp (both CTAs)
    if constexpr (FUSED) {
      comm_warp_run(p.comm, p.num_comm_ops, p.counters + p.num_waves, p.signal_value,
                    reinterpret_cast<char*>(ring), comm_bar, abort_word, p.timeout_ns, lane);
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
    // The four warps walk the same static list of work items to its end (no early exit), so the
    // named barriers they meet at always see all of them.
    const int q = warp & 3;
    PairCursor cur;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool first = true;
    int done_wave = -1;
    uint32_t done_tiles = 0;  // 128-row pieces of this CTA finished in `done_wave`
    uint8_t* wstage = ring + q * (2 * EPI_STAGE_BYTES);
    uint32_t nstore = 0;  // TMA stores this warp has issued
    auto flush_wave = [&]() {
      if constexpr (FUSED) {
        if (done_wave >= 0 && done_tiles > 0) {
          const GemmWave& dw = p.waves[done_wave];
          if (lane == 0) {
            bulk_wait<0>();
            fence_proxy_async();
          }
          __threadfence_system();
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (warp == 4 && lane == 0) {
            // the wave's total in 128-row pieces: every CTA of every pair counts its own
            const uint32_t tiles_w = static_cast<uint32_t>(dw.tiles_m) * static_cast<uint32_t>(dw.tiles_n);
            __threadfence_system();
            const uint32_t old = atomicAdd(&p.counters[done_wave], done_tiles);
            if (old + done_tiles == tiles_w) {
              p.counters[done_wave] = 0;
              __threadfence_system();
              st_release_sys_u64(p.routes[dw.route].flag, p.signal_value);
            }
          }
        }
      }
      done_wave = -1;
      done_tiles = 0;
    };
    PairWork wk;
    for (int n = 0; pair_work(p, tail, total_pair_tiles, pair_id, num_pairs, n, wk); ++n) {
      int m2_blk, n_blk;
      const bool moved = cur.seek(p, wk.tile, m2_blk, n_blk);
      const GemmWave& wv = p.waves[cur.wave];
      if (done_wave >= 0 && done_wave != cur.wave) flush_wave();
      const int row_base = m2_blk * GEMM2_BM + static_cast<int>(cta_rank) * GEMM_BM + q * 32;
      const int grow = row_base + lane;
      char* out_base = reinterpret_cast<char*>(p.c);
      int out_ld = p.ldc;
      int out_row = grow;
      bool reduce = false;
      int tmap_idx = -1, tmap_y = 0;
      if constexpr (FUSED) {
        if (wv.route >= 0) {
          const GemmRoute& rt = p.routes[wv.route];
          out_base = reinterpret_cast<char*>(rt.base);
          out_ld = rt.ld;
          out_row -= wv.off_m * GEMM_BM;
          reduce = rt.reduce != 0;
          if (rt.tmap >= 0) {
            tmap_idx = rt.tmap;
            tmap_y = rt.tmap_row0 + row_base - wv.off_m * GEMM_BM;
          }
          if (moved || first) {
            if (rt.gate != nullptr) {
              if (lane == 0) flag_wait_ge(rt.gate, rt.gate_value, abort_word, p.timeout_ns);
              __syncwarp();
            }
            if (reduce) {
              // the staged partial sums of this wave's rows: one flag per contributing rank
              const unsigned long long t_wait0 = p.trace != nullptr ? globaltimer_ns() : 0ull;
              if (lane < p.num_red) {
                if (!flag_wait_ge(p.red_flags + rt.red_sig[lane], p.signal_value, abort_word, p.timeout_ns)) {
                  abort_info[0] = cur.wave;
                  abort_info[1] = -2 - lane;
                }
              }
              __syncwarp();
              if (p.trace != nullptr && q == 0 && lane == 0) {
                const unsigned long long t_wait1 = globaltimer_ns();
                atomicMin(&p.trace[2 + 3 * cur.wave], t_wait0);
                atomicMax(&p.trace[3 + 3 * cur.wave], t_wait1);
                atomicAdd(&p.trace[4 + 3 * cur.wave], t_wait1 - t_wait0);
              }
            }
          }
        }
      }
      first = false;
      mbar_wait(&tfull_bar[acc], acc_phase, abort_word, p.timeout_ns);
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * ACC_STRIDE);
      const int col0 = n_blk * BN;
      const bool row_ok = grow < p.M;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        tmem_ld_wait();
        const int col = col0 + c * 32;
        if (wk.is_slice) {
          // K slice of a tail tile: add into the fp32 workspace tile
          const int sl = pair_id % tail.slices;
          float4* w = reinterpret_cast<float4*>(
              tail.ws + ((static_cast<size_t>(wk.tile - tail.first_tile) * tail.slices + sl) * GEMM2_BM +
                         (static_cast<size_t>(cta_rank) * GEMM_BM + q * 32 + lane)) * BN + c * 32);
#pragma unroll
          for (int v = 0; v < 8; ++v)
            __stcg(w + v, make_float4(__uint_as_float(r[v * 4 + 0]), __uint_as_float(r[v * 4 + 1]),
                                      __uint_as_float(r[v * 4 + 2]), __uint_as_float(r[v * 4 + 3])));
          continue;
        }
        if constexpr (FUSED) {
          if (reduce && row_ok) epi_add_staged(p, r, grow, col);
        }
        uint4 packed[4];
        epi_pack(r, packed, p.dtype);
        bool staged = false;
        if constexpr (FUSED) {
          if (tmap_idx >= 0) {
            staged = true;
            epi_stage_chunk(wstage, c, lane, packed, &p.tmap_out[tmap_idx], col0, tmap_y, nstore);
          }
        }
        if (!staged && row_ok) {
          uint4* dst = reinterpret_cast<uint4*>(out_base + (static_cast<size_t>(out_row) * out_ld + col) * 2);
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            if (col + v * 8 < p.N) dst[v] = packed[v];
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty_bar[acc]), 0));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
      if constexpr (FUSED) {
        if (wv.route >= 0 && p.routes[wv.route].flag != nullptr) {
          done_wave = cur.wave;
          ++done_tiles;
        }
      }
      if (wk.is_slice) {
        // arrive; wait (bounded) for the tile's other slices; reduce this CTA's share of the rows
        const int tl = wk.tile - tail.first_tile;
        const unsigned int parties = 2u * static_cast<unsigned int>(tail.slices);
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (warp == 4 && lane == 0) {
          atomicAdd(&tail.count[2 * tl], 1u);
          const uint64_t t0 = globaltimer_ns();
          while (ld_acquire_gpu_u32(&tail.count[2 * tl]) < parties) {
            if (*abort_word != 0) break;
            if (globaltimer_ns() - t0 > p.timeout_ns) {
              *abort_word = SYN_DEV_TIMEOUT_COUNTER;
              break;
            }
            __nanosleep(32);
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        __threadfence();
        const int me = (pair_id % tail.slices) * 2 + static_cast<int>(cta_rank);   // 0 .. parties-1
        const int r_lo = GEMM2_BM * me / static_cast<int>(parties), r_hi = GEMM2_BM * (me + 1) / static_cast<int>(parties);
        const int t128 = (warp - 4) * 32 + lane;
        const size_t slice_stride = static_cast<size_t>(GEMM2_BM) * BN;
        for (int idx = t128; idx < (r_hi - r_lo) * (BN / 8); idx += 128) {
          const int rr = r_lo + idx / (BN / 8), cc = idx % (BN / 8);
          const float* base = tail.ws + (static_cast<size_t>(tl) * tail.slices * GEMM2_BM + rr) * BN + cc * 8;
          float acc8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          for (int sidx = 0; sidx < tail.slices; ++sidx) {
            const float4 x = __ldcg(reinterpret_cast<const float4*>(base + sidx * slice_stride));
            const float4 y = __ldcg(reinterpret_cast<const float4*>(base + sidx * slice_stride) + 1);
            acc8[0] += x.x; acc8[1] += x.y; acc8[2] += x.z; acc8[3] += x.w;
            acc8[4] += y.x; acc8[5] += y.y; acc8[6] += y.z; acc8[7] += y.w;
          }
          const int out_r = m2_blk * GEMM2_BM + rr, col = col0 + cc * 8;
          if (out_r < p.M && col < p.N) {
            uint4 u;
            u.x = pack2(acc8[0], acc8[1], p.dtype);
            u.y = pack2(acc8[2], acc8[3], p.dtype);
            u.z = pack2(acc8[4], acc8[5], p.dtype);
            u.w = pack2(acc8[6], acc8[7], p.dtype);
            *reinterpret_cast<uint4*>(reinterpret_cast<char*>(p.c) + (static_cast<size_t>(out_r) * p.ldc + col) * 2) = u;
          }
        }
        // the last CTA to finish reading rewinds the tile's counters for the next launch (every
        // CTA of a slice arrives and departs exactly once on every path, so they always rewind)
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (warp == 4 && lane == 0) {
          const unsigned int old = atomicAdd(&tail.count[2 * tl + 1], 1u);
          if (old == parties - 1u) {
            tail.count[2 * tl] = 0;
            tail.count[2 * tl + 1] = 0;
          }
        }
      }
    }
    flush_wave();
    if constexpr (FUSED) {
      if (lane == 0) bulk_wait<0>();
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // nobody leaves while the peer may still signal this CTA's barriers
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
  if (p.trace != nullptr && threadIdx.x == 0) atomicMax(&p.trace[1], globaltimer_ns());
  if (threadIdx.x == 0 && *abort_word != 0 && p.status != nullptr) {
    if (atomicCAS(p.status, 0, *abort_word) == 0) {
      p.status[1] = abort_info[0];
      p.status[2] = abort_info[1];
      p.status[3] = static_cast<int>(blockIdx.x);
    }
  }
  if constexpr (FUSED) {
    if (threadIdx.x == 0 && *abort_word != 0) {
      for (int w = 0; w < p.num_waves; ++w) {
        const int r = p.waves[w].route;
        if (r >= 0 && p.routes[r].flag != nullptr && p.routes[r].raise_on_abort)
          st_release_sys_u64(p.routes[r].flag, p.signal_value);
      }
    }
  }
}

}  // namespace syn
