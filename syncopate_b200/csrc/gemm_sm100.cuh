// Persistent, warp-specialised bf16/fp16 GEMM for sm_100a: TMA-fed shared-memory ring,
// tcgen05.mma with fp32 accumulators double-buffered in tensor memory, wave-ordered tile
// scheduler with signal flags, optional in-kernel communication:
//   * comm warp: every CTA copies its share of each scheduled chunk between peer-mapped
//     buffers with bulk async copies and publishes a per-chunk flag (all-gather + GEMM),
//   * routed epilogue: a wave's tiles are stored to a peer's staging slab and the peer's flag
//     is raised after the wave's last tile; the wave that owns the local slab adds the staged
//     partial sums in fp32 before storing (GEMM + reduce-scatter).
//
// Behaviour follows Syncopate's Triton templates: consumer wait per wave
// (syncopate/computation/gemm/template.py:90-128), producer counter + notify (:343-348),
// grouped raster inside a wave (:10-18, :130-136).
#pragma once
#include "ptx.cuh"

namespace syn {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;          // 64 x 16-bit = one 128-byte swizzle row
constexpr int GEMM_UMMA_K = 16;
constexpr int GEMM_MAX_WAVES = 64;
constexpr int GEMM_MAX_COMM_OPS = 64;
constexpr int TILE_Q = 4;             // depth of the in-CTA tile queue
constexpr int GEMM_THREADS = 256;    // warp0 TMA, warp1 MMA, warp2 TMEM alloc, warp3 comm, warps4-7 epilogue
#ifndef SYN_COMM_PIECE
#define SYN_COMM_PIECE 8192
#endif
#ifndef SYN_COMM_NBUF
#define SYN_COMM_NBUF 4
#endif
constexpr int COMM_PIECE = SYN_COMM_PIECE;  // bytes per bulk copy of the comm warp
constexpr int COMM_NBUF = SYN_COMM_NBUF;    // ring slots (NBUF - 1 loads in flight at most)
constexpr int EPI_STAGE_BYTES = 32 * 128;     // one epilogue warp's 32 rows x 64 columns of 16 bit
static_assert(COMM_PIECE * COMM_NBUF >= 4 * 2 * EPI_STAGE_BYTES,
              "the routed epilogue stages two 32 x 64 16-bit pieces per epilogue warp there");
constexpr int GEMM_MAX_RED = 7;               // staged partial slabs an owner wave can add (world - 1)
constexpr int GEMM_MAX_KGATES = 16;           // K ranges of A that arrive separately (all-to-all + GEMM)

struct GemmWave {
  int16_t tiles_m, tiles_n;  // tile grid of the wave
  int16_t off_m, off_n;      // first tile of the wave (tile units)
  int16_t csig;              // consumer flag index, -1 = none
  int16_t route;             // index into GemmParams::routes, -1 = plain local store
  int32_t cum;               // tiles in waves [0, w]
};

// Where the tiles of a wave go, and what to raise when the wave is complete.
struct GemmRoute {
  void* base;             // address of element (row off_m*BM, col 0) of the wave in the destination
  uint64_t* flag;         // raised to `signal_value` after the last tile (local or peer memory); may be null
  const uint64_t* gate;   // flag that must be >= gate_value before the first store of the wave; may be null
  uint64_t gate_value;
  int32_t ld;             // destination leading dimension (elements)
  int16_t reduce;         // 1 = add the staged partial sums (reduce-scatter owner wave)
  int16_t tmap;           // index into GemmParams::tmap_out: tiles leave through shared memory and TMA
                          // stores (full 128-byte lines, the form NVLink carries well); -1 = direct stores
  int32_t tmap_row0;      // row of the wave's first tile row in that map's coordinates
  int16_t red_sig[GEMM_MAX_RED];  // reduce waves: flag index (in GemmParams::red_flags) guarding the rows of this
                                  // wave in staged slab s
  int16_t raise_on_abort;  // 1: the flag is local and somebody may wait for it without a bound of its own (a stream
                           // memory operation): a CTA that gave up raises it before it leaves
};

// One 2-D strided copy between mapped buffers, executed cooperatively by all comm warps.
struct CommOp {
  const char* src;
  char* dst;
  uint64_t src_pitch, dst_pitch;
  uint32_t rows, row_bytes;
  const uint64_t* wait_flag;  // local flag that must be >= signal_value before the copy; may be null
  uint64_t* set_flag;         // raised after every CTA's share has landed; may be null
};

struct GemmParams {
  CUtensorMap tmap_a;
  CUtensorMap tmap_b;
  CUtensorMap tmap_out[8];  // destinations of TMA-store routes (one per target rank)
  void* c;
  int32_t ldc;
  int32_t M, N, K;
  int32_t k_blocks;
  int32_t dtype;          // 0 fp16, 1 bf16
  uint32_t idesc;
  int32_t group_m;
  int32_t total_tiles;
  int32_t num_waves;
  int32_t num_comm_ops;
  int32_t num_red;        // staged partial slabs to add in `reduce` routes
  int32_t red_ld;
  int32_t red_row0;       // global C row of the staged slabs' row 0
  const uint64_t* csig;   // consumer flags
  uint32_t* counters;     // [num_waves] producer counters then [num_comm_ops] comm counters, self-resetting
  uint32_t* sched;        // [2] {next tile, CTAs finished}: dynamic tile scheduling when non-null (self-resetting)
  unsigned long long* trace;  // optional [2 + 3 * num_waves] globaltimer stamps: kernel first start / last end,
                              // per wave: earliest flag-wait begin, latest flag-wait end, summed wait ns
  uint64_t signal_value;
  uint64_t timeout_ns;
  int32_t* status;
  // K gates (all-to-all + GEMM): A arrives as ranges of K, each with a flag; every tile walks the
  // ranges in arrival order and waits for a range's flag before its first load from it
  int32_t num_kgates;                 // 0 = K is walked front to back, ungated
  int16_t kgate_kb0[GEMM_MAX_KGATES], kgate_kb1[GEMM_MAX_KGATES];  // k-block range [kb0, kb1)
  int16_t kgate_sig[GEMM_MAX_KGATES]; // consumer flag index, -1 = resident
  const void* red_src[GEMM_MAX_RED];  // staged slabs (address of the slab's row 0)
  const uint64_t* red_flags;          // local flag array the reduce waves' red_sig index
  GemmWave waves[GEMM_MAX_WAVES];
  GemmRoute routes[GEMM_MAX_WAVES];
  CommOp comm[GEMM_MAX_COMM_OPS];
};

struct TileCursor {
  int wave = 0;
  int past = 0;
  // Maps a global tile id (monotone per CTA) to its wave and tile coordinates.
  __device__ __forceinline__ bool seek(const GemmParams& p, int tile, int& m_blk, int& n_blk) {
    bool moved = false;
    while (tile >= p.waves[wave].cum) {
      past = p.waves[wave].cum;
      ++wave;
      moved = true;
    }
    const int local = tile - past;
    const int tm = p.waves[wave].tiles_m, tn = p.waves[wave].tiles_n;
    const int in_group = p.group_m * tn;
    const int group_id = local / in_group;
    const int first_m = group_id * p.group_m;
    const int gsz = min(tm - first_m, p.group_m);
    const int r = local - group_id * in_group;
    m_blk = first_m + (r % gsz) + p.waves[wave].off_m;
    n_blk = (r / gsz) + p.waves[wave].off_n;
    return moved;
  }
};

template <int BN>
struct GemmSmem {
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
  static constexpr int B_BYTES = BN * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
};

__device__ __forceinline__ uint32_t pack2(float lo, float hi, int dtype) {
  if (dtype == 1) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}
__device__ __forceinline__ float2 unpack2(uint32_t u, int dtype) {
  if (dtype == 1) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
  } else {
    return __half22float2(*reinterpret_cast<__half2*>(&u));
  }
}

// Bounded wait (regardless of the abort word) until the phase `parity` of a barrier that counts
// bulk-load bytes has completed: used by a role that gives up while its loads are still in flight,
// because a CTA must not exit while the async proxy may still write its shared memory.
__device__ __forceinline__ void drain_wait(uint64_t* bar, uint32_t parity, uint64_t timeout_ns) {
  const uint64_t t0 = globaltimer_ns();
  while (!mbar_try_wait(bar, parity)) {
    if (globaltimer_ns() - t0 > timeout_ns) break;
  }
}

// The comm warp of each CTA: walks the op list in order; for each op copies pieces
// blockIdx.x, blockIdx.x + gridDim.x, ... through a small shared-memory ring.  A wait that fails
// (its own flag wait, or the CTA's abort word seen inside a ring wait) ends the walk: the loads in
// flight are waited for, nothing more is copied and no flag is raised for the unfinished op.
__device__ __forceinline__ void comm_warp_run(const CommOp* ops, int num_ops, uint32_t* counters,
                                              uint64_t signal_value, char* ring, uint64_t* bars,
                                              volatile int* abort_word, uint64_t timeout_ns, int lane) {
  if (lane != 0) return;
  uint32_t issued = 0;    // loads issued so far, over all ops (ring slot = n % NBUF, parity = (n / NBUF) & 1)
  uint32_t consumed = 0;  // stores issued so far, over all ops (same order as the loads)
  bool ok = true;
  for (int o = 0; o < num_ops && ok; ++o) {
    const CommOp& op = ops[o];
    if (op.wait_flag != nullptr && !flag_wait_ge(op.wait_flag, signal_value, abort_word, timeout_ns)) {
      ok = false;
      break;
    }
    const uint32_t ppr = (op.row_bytes + COMM_PIECE - 1) / COMM_PIECE;
    const uint32_t total = op.rows * ppr;
    constexpr uint32_t LOOKAHEAD = COMM_NBUF - 2;
    uint32_t next_load = blockIdx.x;  // piece index of the next load to issue
    uint32_t cur = blockIdx.x;        // piece index of the next store to issue
    auto issue_load = [&](uint32_t piece) {
      const uint32_t row = piece / ppr, col = (piece - row * ppr) * COMM_PIECE;
      const uint32_t bytes = min(static_cast<uint32_t>(COMM_PIECE), op.row_bytes - col);
      const uint32_t slot = issued % COMM_NBUF;
      mbar_expect_tx(&bars[slot], bytes);
      bulk_g2s(ring + slot * COMM_PIECE, op.src + row * op.src_pitch + col, bytes, &bars[slot]);
      ++issued;
    };
    while (issued - consumed < LOOKAHEAD && next_load < total) {
      issue_load(next_load);
      next_load += gridDim.x;
    }
    while (cur < total) {
      if (next_load < total) {
        // the slot about to be refilled was last read by a store at least two groups back
        bulk_wait_read<1>();
        issue_load(next_load);
        next_load += gridDim.x;
      }
      const uint32_t slot = consumed % COMM_NBUF;
      if (!mbar_wait(&bars[slot], (consumed / COMM_NBUF) & 1u, abort_word, timeout_ns)) {
        ok = false;
        break;
      }
      const uint32_t row = cur / ppr, col = (cur - row * ppr) * COMM_PIECE;
      const uint32_t bytes = min(static_cast<uint32_t>(COMM_PIECE), op.row_bytes - col);
      bulk_s2g(op.dst + row * op.dst_pitch + col, ring + slot * COMM_PIECE, bytes);
      bulk_commit();
      ++consumed;
      cur += gridDim.x;
    }
    if (!ok) break;
    bulk_wait<0>();
    fence_proxy_async();
    if (op.set_flag != nullptr) {
      __threadfence_system();
      const uint32_t old = atomicAdd(&counters[o], 1u);
      if (old == gridDim.x - 1) {
        counters[o] = 0;
        __threadfence_system();
        st_release_sys_u64(op.set_flag, signal_value);
      }
    }
  }
  if (!ok) {
    for (uint32_t n = consumed; n < issued; ++n) drain_wait(&bars[n % COMM_NBUF], (n / COMM_NBUF) & 1u, timeout_ns);
    bulk_wait<0>();
  }
}

// Bounded wait for the bulk loads still in flight into one stage of this CTA's shared memory, for a
// producer that gives up: a CTA must not exit while the async proxy may still write its shared
// memory.  `fills` = how many times the stage's full barrier has been armed with a load.
__device__ __forceinline__ void drain_stage(uint64_t* full_bar, uint32_t fills, uint64_t timeout_ns) {
  if (fills != 0) drain_wait(full_bar, (fills - 1u) & 1u, timeout_ns);
}

// Adds the 16-bit partial sums staged by the peers (slab order = rank order, fixed) to 32 fp32
// accumulator values of one output row.  The loads of all slabs are issued before the first add:
// the rows are 16 KB or more apart, so the reads are latency-bound and one round trip per chunk
// of columns is what the epilogue pays.
__device__ __forceinline__ void epi_add_staged(const GemmParams& p, uint32_t (&r)[32], int grow, int col) {
  const size_t elem = static_cast<size_t>(grow - p.red_row0) * p.red_ld + col;
  uint4 u[GEMM_MAX_RED][4];
#pragma unroll
  for (int s = 0; s < GEMM_MAX_RED; ++s) {
    if (s < p.num_red) {
      const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(p.red_src[s]) + elem * 2);
#pragma unroll
      for (int v = 0; v < 4; ++v)
        if (col + v * 8 < p.N) u[s][v] = __ldcg(src + v);
    }
  }
#pragma unroll
  for (int s = 0; s < GEMM_MAX_RED; ++s) {
    if (s < p.num_red) {
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        if (col + v * 8 < p.N) {
          const uint32_t w4[4] = {u[s][v].x, u[s][v].y, u[s][v].z, u[s][v].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = unpack2(w4[j], p.dtype);
            r[v * 8 + 2 * j] = __float_as_uint(__uint_as_float(r[v * 8 + 2 * j]) + f.x);
            r[v * 8 + 2 * j + 1] = __float_as_uint(__uint_as_float(r[v * 8 + 2 * j + 1]) + f.y);
          }
        }
      }
    }
  }
}

__device__ __forceinline__ void epi_pack(const uint32_t (&r)[32], uint4 (&packed)[4], int dtype) {
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    packed[v].x = pack2(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1]), dtype);
    packed[v].y = pack2(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]), dtype);
    packed[v].z = pack2(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]), dtype);
    packed[v].w = pack2(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]), dtype);
  }
}

// TMA-store route, one epilogue warp: the warp's 32 rows of a 64-column half tile go through one of
// the warp's own two 4 KB staging pieces (128-byte swizzle of the output tensor map) and leave as
// one 32 x 64 box issued by the warp's lane 0.  No other warp is involved, so nothing but the warp
// itself synchronises.  `c` is the index of the 32-column chunk inside the tile.
__device__ __forceinline__ void epi_stage_chunk(uint8_t* wstage, int c, int lane, const uint4 (&packed)[4],
                                                const CUtensorMap* map, int x0, int y, uint32_t& nstore) {
  // the two pieces alternate with the stores this warp has issued (over tiles as well), so the
  // piece being refilled was read by the store before the previous one
  uint8_t* sbuf = wstage + (nstore & 1u) * EPI_STAGE_BYTES;
  if ((c & 1) == 0) {
    if (lane == 0) bulk_wait_read<1>();  // the store that last read this piece is done with it
    __syncwarp();
  }
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    const int chunk16 = (c & 1) * 4 + v;
    *reinterpret_cast<uint4*>(sbuf + lane * 128 + ((chunk16 ^ (lane & 7)) << 4)) = packed[v];
  }
  if (c & 1) {
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      tma_store_2d(map, sbuf, x0 + (c >> 1) * 64, y);
      bulk_commit();
    }
    ++nstore;
  }
}

template <int BN, int STAGES, bool FUSED>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_kernel(const __grid_constant__ GemmParams p) {
  using L = GemmSmem<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * L::A_BYTES;
  uint8_t* ring = smem + STAGES * L::STAGE_BYTES;  // FUSED only
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring + (FUSED ? COMM_NBUF * COMM_PIECE : 0));
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tfull_bar = bars + 2 * STAGES;
  uint64_t* tempty_bar = bars + 2 * STAGES + 2;
  uint64_t* comm_bar = bars + 2 * STAGES + 4;
  uint64_t* tq_full = comm_bar + COMM_NBUF;   // tile queue: producer -> MMA issuer and epilogue
  uint64_t* tq_empty = tq_full + TILE_Q;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tq_empty + TILE_Q);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_holder + 1);
  int* abort_info = const_cast<int*>(abort_word) + 1;  // {wave, flag}
  volatile int* tile_q = reinterpret_cast<volatile int*>(abort_info + 2);  // [TILE_Q] tile ids, -1 = no more
  volatile int* epi_sync = tile_q + TILE_Q;  // [2][2] {tile, abort} agreed on by the four epilogue warps

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = (2 * BN <= 256) ? 256 : 512;
  constexpr int ACC_STRIDE = TMEM_COLS / 2;  // column offset of the second accumulator

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull_bar[i], 1);
      mbar_init(&tempty_bar[i], 4);
    }
    for (int i = 0; i < COMM_NBUF; ++i) mbar_init(&comm_bar[i], 1);
    for (int i = 0; i < TILE_Q; ++i) {
      mbar_init(&tq_full[i], 1);
      mbar_init(&tq_empty[i], 5);  // the MMA thread and one lane of each epilogue warp
    }
    *abort_word = 0;
    abort_info[0] = -1;
    abort_info[1] = -1;
    fence_mbar_init();
  }
  if (warp == 2) {
    tmem_alloc(tmem_holder, TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tmap(&p.tmap_a);
    prefetch_tmap(&p.tmap_b);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  if (p.trace != nullptr && threadIdx.x == 0) atomicMin(&p.trace[0], globaltimer_ns());

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      TileCursor cur;
      int stage = 0;
      uint32_t phase = 0;
      uint32_t issued = 0;  // k-block loads issued so far
      int gates_passed = 0;  // K ranges whose flag this CTA has seen up
      bool first = true;
      bool gave_up = false;
      for (uint32_t n = 0; !gave_up; ++n) {
        // next tile: taken from the grid-wide counter (dynamic) or round-robin (static), then
        // handed to the other roles through the tile queue
        const int slot = n % TILE_Q;
        mbar_wait(&tq_empty[slot], ((n / TILE_Q) & 1u) ^ 1u, abort_word, p.timeout_ns);
        int tile = p.sched != nullptr ? static_cast<int>(atomicAdd(p.sched, 1u))
                                      : static_cast<int>(blockIdx.x + n * gridDim.x);
        if (tile >= p.total_tiles || *abort_word != 0) tile = -1;
        tile_q[slot] = tile;
        mbar_arrive(&tq_full[slot]);
        if (tile < 0) break;
        int m_blk, n_blk;
        const bool moved = cur.seek(p, tile, m_blk, n_blk);
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
            fence_proxy_async();  // order the flag read before async-proxy (TMA) reads of the chunk
            if (p.trace != nullptr) {
              const unsigned long long t_wait1 = globaltimer_ns();
              atomicMin(&p.trace[2 + 3 * cur.wave], t_wait0);
              atomicMax(&p.trace[3 + 3 * cur.wave], t_wait1);
              atomicAdd(&p.trace[4 + 3 * cur.wave], t_wait1 - t_wait0);
            }
          }
          first = false;
        }
        const int ranges = p.num_kgates > 0 ? p.num_kgates : 1;
        for (int g = 0; g < ranges && !gave_up; ++g) {
          int kb_lo = 0, kb_hi = p.k_blocks;
          if (p.num_kgates > 0) {
            kb_lo = p.kgate_kb0[g];
            kb_hi = p.kgate_kb1[g];
            if (g >= gates_passed) {
              // first tile of this CTA that reaches the range: its flag must be up
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
              gave_up = true;  // somebody in the CTA gave up: the stage may never be released
              break;
            }
            mbar_expect_tx(&full_bar[stage], L::STAGE_BYTES);
            tma_load_2d(sA + stage * L::A_BYTES, &p.tmap_a, &full_bar[stage], kb * GEMM_BK, m_blk * GEMM_BM);
            tma_load_2d(sB + stage * L::B_BYTES, &p.tmap_b, &full_bar[stage], kb * GEMM_BK, n_blk * BN);
            ++issued;
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
      }
      if (*abort_word != 0) {
        // loads already issued keep writing this CTA's shared memory: wait for them before leaving
        for (int s = 0; s < STAGES; ++s)
          drain_stage(&full_bar[s], issued / STAGES + (static_cast<uint32_t>(s) < issued % STAGES ? 1u : 0u), p.timeout_ns);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // The whole warp walks the tiles and waits on the barriers; one elected lane issues each
    // tcgen05 instruction (and makes the queue hand-back).
    {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      const uint32_t desc_hi = static_cast<uint32_t>(make_smem_desc_sw128(0, 16, 1024) >> 32);
      const uint32_t a_lo0 = static_cast<uint32_t>(make_smem_desc_sw128(smem_u32(sA), 16, 1024));
      const uint32_t b_lo0 = static_cast<uint32_t>(make_smem_desc_sw128(smem_u32(sB), 16, 1024));
      const uint32_t idesc = p.idesc;
      const int k_blocks = p.k_blocks;
      const uint64_t timeout_ns = p.timeout_ns;
      for (uint32_t n = 0;; ++n) {
        const int slot = n % TILE_Q;
        mbar_wait(&tq_full[slot], (n / TILE_Q) & 1u, abort_word, timeout_ns);
        const int tile = tile_q[slot];
        __syncwarp();  // every lane has read the slot before it is handed back
        if (elect_one()) mbar_arrive(&tq_empty[slot]);
        if (tile < 0 || *abort_word != 0) break;
        mbar_wait(&tempty_bar[acc], acc_phase ^ 1u, abort_word, timeout_ns);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * ACC_STRIDE);
        for (int kb = 0; kb < k_blocks; ++kb) {
          mbar_wait(&full_bar[stage], phase, abort_word, timeout_ns);
          tc_fence_after();
          const uint32_t a_lo = a_lo0 + static_cast<uint32_t>(stage) * (L::A_BYTES >> 4);
          const uint32_t b_lo = b_lo0 + static_cast<uint32_t>(stage) * (L::B_BYTES >> 4);
#pragma unroll
          for (int k = 0; k < GEMM_BK / GEMM_UMMA_K; ++k) {
            // advancing 16 elements along K inside the 128-byte swizzle row = +32 bytes = +2 (16-byte units)
            if (elect_one())
              umma_ss_words(d_tmem, a_lo + 2u * k, desc_hi, b_lo + 2u * k, desc_hi, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          if (elect_one()) umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (elect_one()) umma_commit(&tfull_bar[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else if (warp == 3) {
    // ------------------------------------------------------------ comm warp
    if constexpr (FUSED) {
      comm_warp_run(p.comm, p.num_comm_ops, p.counters + p.num_waves, p.signal_value,
                    reinterpret_cast<char*>(ring), comm_bar, abort_word, p.timeout_ns, lane);
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------ epilogue (TMEM -> registers -> global)
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    TileCursor cur;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool first = true;
    int done_wave = -1;        // wave whose tiles this CTA has stored but not yet counted
    uint32_t done_tiles = 0;
    uint8_t* wstage = ring + q * (2 * EPI_STAGE_BYTES);  // this warp's staging pieces (TMA-store routes)
    uint32_t nstore = 0;                                  // TMA stores this warp has issued
    // counts this CTA's finished tiles of a wave once, when it leaves the wave: every warp's TMA
    // stores have been performed and its plain stores fenced before the count; the CTA that
    // completes the wave's total raises the wave's flag
    auto flush_wave = [&]() {
      if constexpr (FUSED) {
        if (done_wave >= 0 && done_tiles > 0) {
          const GemmWave& dw = p.waves[done_wave];
          if (lane == 0) {
            bulk_wait<0>();
            fence_proxy_async();
          }
          __threadfence_system();
          asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps
          if (warp == 4 && lane == 0) {
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
    for (uint32_t n = 0;; ++n) {
      const int slot = n % TILE_Q;
      mbar_wait(&tq_full[slot], (n / TILE_Q) & 1u, abort_word, p.timeout_ns);
      int tile = tile_q[slot];
      int ab = *abort_word;
      __syncwarp();
      if (lane == 0) mbar_arrive(&tq_empty[slot]);
      if constexpr (FUSED) {
        // The four warps meet at named barriers inside a wave (flush_wave): they must take the
        // same tiles and leave at the same tile, so warp 4's view of the queue slot and of the
        // abort word is the one all of them use.
        if (warp == 4 && lane == 0) {
          epi_sync[2 * (n & 1u)] = tile;
          epi_sync[2 * (n & 1u) + 1] = ab;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        tile = epi_sync[2 * (n & 1u)];
        ab = epi_sync[2 * (n & 1u) + 1];
      }
      if (tile < 0 || tile >= p.total_tiles || ab != 0) break;
      int m_blk, n_blk;
      const bool moved = cur.seek(p, tile, m_blk, n_blk);
      const GemmWave& wv = p.waves[cur.wave];
      if (done_wave >= 0 && done_wave != cur.wave) flush_wave();
      // destination of this tile
      char* out_base = reinterpret_cast<char*>(p.c);
      int out_ld = p.ldc;
      int out_row = m_blk * GEMM_BM + q * 32 + lane;  // row inside the destination
      const int grow = out_row;                       // global row of C
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
            tmap_y = rt.tmap_row0 + (m_blk - wv.off_m) * GEMM_BM + q * 32;
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
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;

      if constexpr (FUSED) {
        if (wv.route >= 0 && p.routes[wv.route].flag != nullptr) {
          done_wave = cur.wave;
          ++done_tiles;
        }
      }
    }
    flush_wave();
    if constexpr (FUSED) {
      if (lane == 0) bulk_wait<0>();  // staged pieces still being read by this warp's TMA stores
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (p.trace != nullptr && threadIdx.x == 0) atomicMax(&p.trace[1], globaltimer_ns());
  if (threadIdx.x == 0 && p.sched != nullptr) {
    // the last CTA to get here (every CTA has stopped taking tiles by then) rewinds the scheduler
    const uint32_t old = atomicAdd(&p.sched[1], 1u);
    if (old == gridDim.x - 1) {
      p.sched[0] = 0;
      p.sched[1] = 0;
    }
  }
  if (threadIdx.x == 0 && *abort_word != 0 && p.status != nullptr) {
    if (atomicCAS(p.status, 0, *abort_word) == 0) {
      p.status[1] = abort_info[0];
      p.status[2] = abort_info[1];
      p.status[3] = static_cast<int>(blockIdx.x);
    }
  }
  if constexpr (FUSED) {
    // Somebody outside the kernel may be waiting for the wave flags without a bound of its own (a
    // stream memory operation): after a failed wait the data are lost anyway, so let everybody go on.
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
