// Host side of the fused operators: turns lowered schedules plus symmetric-buffer tables into the
// comm-op list and the routed-epilogue table of the persistent GEMM kernel.
#include <algorithm>
#include <vector>

#include "gemm_host.h"

#include <stdlib.h>

namespace syn {

// SYNCOPATE_B200_STATIC_SCHED=1 keeps the round-robin tile order in the fused kernels (tuning aid).
static bool dynamic_sched() {
  static int cached = -1;
  if (cached < 0) {
    const char* e = getenv("SYNCOPATE_B200_STATIC_SCHED");
    cached = (e != nullptr && e[0] == '1') ? 0 : 1;
  }
  return cached == 1;
}

static int check_symm(const syn_symm& s) {
  if (s.world <= 0 || s.world > SYN_MAX_WORLD || s.rank < 0 || s.rank >= s.world) return SYN_ERR_INVALID;
  for (int r = 0; r < s.world; ++r)
    if (s.ptrs[r] == nullptr) return SYN_ERR_INVALID;
  return SYN_OK;
}


// Reduce pass of GEMM + reduce-scatter: out[rows, N] (the rank's own 16-bit partial sums, stored by
// the GEMM) += the partial sums the other ranks staged, in fp32, fixed slab order.  A stand-alone
// pass reads whole 128-byte lines with coalesced 16-byte loads, which the routed epilogue (one
// thread per accumulator row, rows 16 KB apart) cannot; it costs a launch and one more rounding of
// the own partial sum to 16 bits, the rounding every other rank's partial sum gets anyway.
struct RsReduceParams {
  void* out;              // row 0 of the piece
  int ldo, rows, n_vec;   // n_vec = N / 8
  int num_red, dtype;
  const void* src[GEMM_MAX_RED];  // row 0 of the piece in each staged slab
  int src_ld;
  const uint64_t* flags;
  int16_t sig[GEMM_MAX_RED];
  uint64_t value, timeout_ns;
  int32_t* status;
  int wave;
};

__global__ void __launch_bounds__(256) rs_reduce_kernel(const RsReduceParams p) {
  __shared__ int abort_word;
  if (threadIdx.x == 0) abort_word = 0;
  __syncthreads();
  if (threadIdx.x < p.num_red) {
    volatile int* aw = &abort_word;
    if (!flag_wait_ge(p.flags + p.sig[threadIdx.x], p.value, aw, p.timeout_ns) && p.status != nullptr) {
      if (atomicCAS(p.status, 0, SYN_DEV_TIMEOUT_FLAG) == 0) {
        p.status[1] = p.wave;
        p.status[2] = -2 - static_cast<int>(threadIdx.x);
        p.status[3] = static_cast<int>(blockIdx.x);
      }
    }
  }
  __syncthreads();
  if (abort_word != 0) return;  // the rows keep the own partial sum; the error is in the status block
  const size_t total = static_cast<size_t>(p.rows) * p.n_vec;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t row = i / p.n_vec, v = i % p.n_vec;
    uint4* dst = reinterpret_cast<uint4*>(static_cast<char*>(p.out) + (row * p.ldo + v * 8) * 2);
    uint4 u[GEMM_MAX_RED];
    const uint4 own = *dst;
#pragma unroll
    for (int s = 0; s < GEMM_MAX_RED; ++s)
      if (s < p.num_red)
        u[s] = __ldcs(reinterpret_cast<const uint4*>(static_cast<const char*>(p.src[s]) + (row * p.src_ld + v * 8) * 2));
    const uint32_t o4[4] = {own.x, own.y, own.z, own.w};
    float2 acc[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[j] = unpack2(o4[j], p.dtype);
#pragma unroll
    for (int s = 0; s < GEMM_MAX_RED; ++s) {
      if (s < p.num_red) {
        const uint32_t w4[4] = {u[s].x, u[s].y, u[s].z, u[s].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack2(w4[j], p.dtype);
          acc[j].x += f.x;
          acc[j].y += f.y;
        }
      }
    }
    uint4 r;
    r.x = pack2(acc[0].x, acc[0].y, p.dtype);
    r.y = pack2(acc[1].x, acc[1].y, p.dtype);
    r.z = pack2(acc[2].x, acc[2].y, p.dtype);
    r.w = pack2(acc[3].x, acc[3].y, p.dtype);
    *dst = r;
  }
}

int preload_fused_kernels() {
  cudaFuncAttributes attr;
  SYN_CUDA_TRY(cudaFuncGetAttributes(&attr, rs_reduce_kernel));
  return SYN_OK;
}

}  // namespace syn

extern "C" {

int syn_ag_gemm(const syn_ag_gemm_args* args, const syn_schedule* a_sched, void* stream) {
  using namespace syn;
  if (args == nullptr || a_sched == nullptr) return SYN_ERR_INVALID;
  const syn_gemm_args& g = args->gemm;
  int rc = check_symm(args->a);
  if (rc != SYN_OK) return rc;
  if (a_sched->ndim != 2 || a_sched->num_waves <= 0 || a_sched->num_waves > GEMM_MAX_WAVES) return SYN_ERR_INVALID;
  if (a_sched->offsets == nullptr || a_sched->shapes == nullptr) return SYN_ERR_INVALID;
  if (args->a.ptrs[args->a.rank] != g.a) return SYN_ERR_INVALID;  // gemm.a must be the local copy
  const int world = args->a.world, rank = args->a.rank;
  const int lda = g.lda ? g.lda : g.K;
  if (g.M % world != 0) return SYN_ERR_SHAPE;
  const int rows_per_rank = g.M / world;

  // GEMM waves over C: the rows of each A block, all N columns
  const int nw = a_sched->num_waves;
  std::vector<int32_t> c_off(nw * 2), c_shape(nw * 2);
  for (int w = 0; w < nw; ++w) {
    const int r0 = a_sched->offsets[w * 2], k0 = a_sched->offsets[w * 2 + 1];
    const int rows = a_sched->shapes[w * 2], cols = a_sched->shapes[w * 2 + 1];
    if (r0 < 0 || rows <= 0 || r0 + rows > g.M || k0 < 0 || cols <= 0 || k0 + cols > g.K) return SYN_ERR_SHAPE;
    c_off[w * 2] = r0;
    c_off[w * 2 + 1] = 0;
    c_shape[w * 2] = rows;
    c_shape[w * 2 + 1] = g.N;
  }
  syn_schedule c_sched = *a_sched;
  c_sched.offsets = c_off.data();
  c_sched.shapes = c_shape.data();

  int grid = 0, bn = 0;
  bool want_pair = false;
  rc = gemm_resolve_grid_and_bn(&g, &c_sched, &grid, &bn, 32, &want_pair);
  if (rc != SYN_OK) return rc;
  GemmParams p;
  rc = gemm_fill_common(&p, &g, &c_sched, bn);
  if (rc != SYN_OK) return rc;

  // comm ops: one pull per remote block, in wave order
  int n_ops = 0;
  for (int w = 0; w < nw; ++w) {
    const int sig = a_sched->signals ? a_sched->signals[w] : -1;
    const int tgt = a_sched->target_ranks ? a_sched->target_ranks[w] : -1;
    if (sig < 0 || tgt < 0 || tgt == rank) continue;  // resident block
    if (g.consumer_signal_ptr == nullptr || args->counters == nullptr) return SYN_ERR_INVALID;
    if (n_ops >= GEMM_MAX_COMM_OPS) return SYN_ERR_TOO_LARGE;
    const int r0 = a_sched->offsets[w * 2], k0 = a_sched->offsets[w * 2 + 1];
    const int rows = a_sched->shapes[w * 2], cols = a_sched->shapes[w * 2 + 1];
    // the block's owner holds it at the same place of its own copy of the gathered buffer; on an
    // all-to-all fabric a ring plan's block is fetched from its owner too, in the plan's order
    const int owner = r0 / rows_per_rank;
    if (owner < 0 || owner >= world || (r0 + rows - 1) / rows_per_rank != owner) return SYN_ERR_SHAPE;
    if (owner == rank) continue;
    const int pr0 = a_sched->dst_offsets ? a_sched->dst_offsets[w * 2] : r0;
    const int pk0 = a_sched->dst_offsets ? a_sched->dst_offsets[w * 2 + 1] : k0;
    const int src_r0 = (tgt == owner) ? pr0 : r0;
    const int src_k0 = (tgt == owner) ? pk0 : k0;
    CommOp& op = p.comm[n_ops++];
    op.src = static_cast<const char*>(args->a.ptrs[owner]) + (static_cast<size_t>(src_r0) * lda + src_k0) * 2;
    op.dst = static_cast<char*>(const_cast<void*>(g.a)) + (static_cast<size_t>(r0) * lda + k0) * 2;
    if ((reinterpret_cast<uintptr_t>(op.src) & 15) || (reinterpret_cast<uintptr_t>(op.dst) & 15) || (cols % 8))
      return SYN_ERR_INVALID;
    if (cols == lda) {  // contiguous block: one long row
      op.rows = 1;
      op.row_bytes = static_cast<uint32_t>(static_cast<size_t>(rows) * cols * 2);
      if (static_cast<size_t>(rows) * cols * 2 > 0xFFFFFFFFull) return SYN_ERR_TOO_LARGE;
      op.src_pitch = op.dst_pitch = 0;
    } else {
      op.rows = static_cast<uint32_t>(rows);
      op.row_bytes = static_cast<uint32_t>(cols * 2);
      op.src_pitch = op.dst_pitch = static_cast<uint64_t>(lda) * 2;
    }
    op.wait_flag = nullptr;
    op.set_flag = const_cast<uint64_t*>(g.consumer_signal_ptr) + sig;
  }
  p.num_comm_ops = n_ops;
  p.counters = args->counters;
  // the CTA-pair kernel where the waves allow it (256-row boundaries); it hands tiles out round-robin
  if (want_pair && pair_eligible(p, bn, grid))
    return gemm_launch_pair(p, &g, bn, grid, /*fused=*/n_ops > 0, static_cast<cudaStream_t>(stream));
  if (args->counters != nullptr && dynamic_sched()) p.sched = args->counters + SYN_MAX_WAVES + SYN_MAX_COMM_OPS;
  grid = std::min(grid, p.total_tiles);
  if (grid <= 0) return SYN_ERR_INVALID;
  return gemm_launch(p, bn, /*fused=*/n_ops > 0, grid, static_cast<cudaStream_t>(stream));
}

int syn_gemm_rs(const syn_gemm_rs_args* args, const syn_schedule* src_sched, const syn_schedule* dst_sched,
                void* stream) {
  using namespace syn;
  if (args == nullptr || src_sched == nullptr || dst_sched == nullptr) return SYN_ERR_INVALID;
  syn_gemm_args g = args->gemm;
  int rc = check_symm(args->stage);
  if (rc != SYN_OK) return rc;
  rc = check_symm(args->recv_flags);
  if (rc != SYN_OK) return rc;
  const int world = args->stage.world, rank = args->stage.rank;
  if (args->recv_flags.world != world || args->recv_flags.rank != rank) return SYN_ERR_INVALID;
  if (args->out == nullptr || args->counters == nullptr) return SYN_ERR_INVALID;
  if (args->send_buf != nullptr && (args->send_flags == nullptr || (reinterpret_cast<uintptr_t>(args->send_buf) & 15)))
    return SYN_ERR_INVALID;
  if (src_sched->ndim != 2 || src_sched->target_ranks == nullptr || src_sched->num_waves <= 0) return SYN_ERR_INVALID;
  if (src_sched->offsets == nullptr || src_sched->shapes == nullptr) return SYN_ERR_INVALID;
  // the receive buffer is [M / world, N] (direct reduce) or [world, M / world, N] (one slab per sender):
  // rows and columns are its last two axes
  const int dnd = dst_sched->ndim;
  if ((dnd != 2 && dnd != 3) || dst_sched->num_waves <= 0 || dst_sched->offsets == nullptr || dst_sched->shapes == nullptr)
    return SYN_ERR_INVALID;
  if (g.M % world != 0) return SYN_ERR_SHAPE;
  const int slab_rows = g.M / world;
  const int ldo = args->ldo ? args->ldo : g.N;
  if (ldo < g.N || (ldo % 8) || (reinterpret_cast<uintptr_t>(args->out) & 15)) return SYN_ERR_INVALID;
  // the whole partial product is never stored; give the argument check a non-null placeholder
  if (g.c == nullptr) g.c = args->out;
  g.consumer_signal_ptr = nullptr;

  // ---- what arrives here: pieces of this rank's slab staged by the other ranks, one flag each.
  // Pieces are grouped by the rows they cover; a group that every other rank contributes to
  // becomes one reduce wave that waits for exactly its own flags.
  struct Group {
    int off, rows;
    int sig[SYN_MAX_WORLD];
  };
  std::vector<Group> groups;
  int src_index[SYN_MAX_WORLD];  // source rank -> position among the staged slabs
  int n_red = 0;
  for (int r = 0; r < SYN_MAX_WORLD; ++r) src_index[r] = -1;
  for (int w = 0; w < dst_sched->num_waves; ++w) {
    const int src_rank = dst_sched->target_ranks ? dst_sched->target_ranks[w] : -1;
    const int sig = dst_sched->signals ? dst_sched->signals[w] : -1;
    if (src_rank < 0 || src_rank == rank) continue;
    if (src_rank >= world || sig < 0 || sig > 32767) return SYN_ERR_SHAPE;
    if (dst_sched->offsets[w * dnd + dnd - 1] != 0 || dst_sched->shapes[w * dnd + dnd - 1] != g.N) return SYN_ERR_SHAPE;
    if (src_index[src_rank] < 0) {
      if (n_red >= GEMM_MAX_RED) return SYN_ERR_SHAPE;
      src_index[src_rank] = n_red++;
    }
    const int off = dst_sched->offsets[w * dnd + dnd - 2], rows = dst_sched->shapes[w * dnd + dnd - 2];
    Group* grp = nullptr;
    for (auto& x : groups)
      if (x.off == off && x.rows == rows) grp = &x;
    if (grp == nullptr) {
      Group fresh;
      fresh.off = off;
      fresh.rows = rows;
      for (int r = 0; r < SYN_MAX_WORLD; ++r) fresh.sig[r] = -1;
      groups.push_back(fresh);
      grp = &groups.back();
    }
    if (grp->sig[src_index[src_rank]] >= 0) return SYN_ERR_SHAPE;  // the same rows twice from one rank
    grp->sig[src_index[src_rank]] = sig;
  }
  if (n_red != world - 1) return SYN_ERR_SHAPE;
  std::sort(groups.begin(), groups.end(), [](const Group& x, const Group& y) { return x.off < y.off; });
  int covered = 0;
  for (const auto& x : groups) {
    if (x.off != covered || x.rows <= 0 || (x.off % GEMM_BM) != 0) return SYN_ERR_SHAPE;
    for (int i = 0; i < n_red; ++i)
      if (x.sig[i] < 0) return SYN_ERR_SHAPE;  // every other rank contributes to every group
    covered += x.rows;
  }
  if (covered != slab_rows) return SYN_ERR_SHAPE;

  // ---- the waves the kernel walks: those of `src_sched`, with the wave kept here cut into the groups
  struct Piece {
    int r0, rows, orig, group;  // group >= 0: reduce wave
  };
  std::vector<Piece> pieces;
  for (int w = 0; w < src_sched->num_waves; ++w) {
    const int r0 = src_sched->offsets[w * 2], rows = src_sched->shapes[w * 2];
    if (src_sched->offsets[w * 2 + 1] != 0 || src_sched->shapes[w * 2 + 1] != g.N) return SYN_ERR_SHAPE;
    if (r0 < 0 || rows <= 0 || r0 + rows > g.M) return SYN_ERR_SHAPE;
    const int owner = r0 / slab_rows;  // rank whose output the rows belong to
    if ((r0 + rows - 1) / slab_rows != owner) return SYN_ERR_SHAPE;
    int tgt = src_sched->target_ranks[w];
    if (tgt < 0) tgt = rank;
    if (tgt != owner) return SYN_ERR_SHAPE;
    if (tgt != rank) {
      pieces.push_back({r0, rows, w, -1});
      continue;
    }
    const int lo = r0 - rank * slab_rows, hi = lo + rows;
    for (size_t gi = 0; gi < groups.size(); ++gi) {
      const int a = std::max(lo, groups[gi].off), b = std::min(hi, groups[gi].off + groups[gi].rows);
      if (a >= b) continue;
      if (a != groups[gi].off || b != groups[gi].off + groups[gi].rows) return SYN_ERR_SHAPE;  // partial overlap
      pieces.push_back({rank * slab_rows + a, b - a, w, static_cast<int>(gi)});
    }
  }
  const int nw = static_cast<int>(pieces.size());
  if (nw > GEMM_MAX_WAVES) return SYN_ERR_TOO_LARGE;
  std::vector<int32_t> k_off(nw * 2), k_shape(nw * 2), k_sig(nw, -1);
  for (int w = 0; w < nw; ++w) {
    k_off[w * 2] = pieces[w].r0;
    k_off[w * 2 + 1] = 0;
    k_shape[w * 2] = pieces[w].rows;
    k_shape[w * 2 + 1] = g.N;
  }
  syn_schedule k_sched;
  memset(&k_sched, 0, sizeof(k_sched));
  k_sched.num_waves = nw;
  k_sched.ndim = 2;
  k_sched.offsets = k_off.data();
  k_sched.shapes = k_shape.data();
  k_sched.signals = k_sig.data();

  int grid = 0, bn = 0;
  bool want_pair = false;
  rc = gemm_resolve_grid_and_bn(&g, &k_sched, &grid, &bn, /*multiple=*/64, &want_pair);
  if (rc != SYN_OK) return rc;
  GemmParams p;
  rc = gemm_fill_common(&p, &g, &k_sched, bn);
  if (rc != SYN_OK) return rc;
  const uint64_t epoch = p.signal_value;
  int tmap_of_rank[SYN_MAX_WORLD];
  for (int r = 0; r < SYN_MAX_WORLD; ++r) tmap_of_rank[r] = -1;
  int n_maps = 0;
  const size_t slab_elems = static_cast<size_t>(slab_rows) * g.N;
  const size_t half = static_cast<size_t>(epoch & 1) * world;

  for (int w = 0; w < nw; ++w) {
    const Piece& pc = pieces[w];
    const int tgt = pc.r0 / slab_rows;
    GemmRoute& rt = p.routes[w];
    p.waves[w].route = static_cast<int16_t>(w);
    rt.gate = nullptr;
    rt.gate_value = 0;
    const int row_in_slab = pc.r0 - tgt * slab_rows;
    char* slab0;  // row 0 of the destination slab
    int slab_ld;
    bool local = true;
    if (tgt == rank) {
      slab0 = static_cast<char*>(args->out);
      slab_ld = ldo;
      if (args->reduce_pass) {
        // plain store of the own partial sum; the pass behind the kernel adds the staged ones
        rt.flag = nullptr;
        rt.reduce = 0;
      } else {
        rt.flag = args->out_flags != nullptr ? args->out_flags + pc.group : nullptr;
        rt.raise_on_abort = 1;
        rt.reduce = 1;
        for (int i = 0; i < n_red; ++i) rt.red_sig[i] = static_cast<int16_t>(groups[pc.group].sig[i]);
      }
    } else if (args->send_buf != nullptr) {
      // transport by the caller: local send slab, local flag per wave
      slab0 = static_cast<char*>(args->send_buf) + static_cast<size_t>(tgt) * slab_elems * 2;
      slab_ld = g.N;
      rt.flag = args->send_flags + pc.orig;
      rt.raise_on_abort = 1;
      rt.reduce = 0;
    } else {
      slab0 = static_cast<char*>(args->stage.ptrs[tgt]) + (half + rank) * slab_elems * 2;
      slab_ld = g.N;
      const int rsig = args->remote_signals ? args->remote_signals[pc.orig] : -1;
      rt.flag = rsig >= 0 ? static_cast<uint64_t*>(args->recv_flags.ptrs[tgt]) + rsig : nullptr;
      rt.reduce = 0;
      local = false;
    }
    rt.base = slab0 + static_cast<size_t>(row_in_slab) * slab_ld * 2;
    rt.ld = slab_ld;
    rt.tmap = -1;
    rt.tmap_row0 = row_in_slab;
    if (!local) {
      // tiles for a peer leave through shared memory and TMA stores (full 128-byte lines): one
      // output map per destination slab, boxes of one epilogue warp's 32 rows x 64 columns
      if (tmap_of_rank[tgt] < 0) {
        rc = encode_tmap_2d_sw128(&p.tmap_out[n_maps], slab0, slab_rows, g.N, slab_ld, 32, 64);
        if (rc != SYN_OK) return rc;
        tmap_of_rank[tgt] = n_maps++;
      }
      rt.tmap = static_cast<int16_t>(tmap_of_rank[tgt]);
    }
  }
  // staged partial sums, in the order of `src_index`, and the flag array the reduce waves index
  for (int r = 0; r < world; ++r)
    if (src_index[r] >= 0)
      p.red_src[src_index[r]] = static_cast<const char*>(args->stage.ptrs[rank]) + (half + r) * slab_elems * 2;
  p.red_flags = static_cast<const uint64_t*>(args->recv_flags.ptrs[rank]);
  p.num_red = n_red;
  p.red_ld = g.N;
  p.red_row0 = rank * slab_rows;
  p.counters = args->counters;
  p.c = args->out;
  p.ldc = ldo;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  if (want_pair && pair_eligible(p, bn, grid)) {
    rc = gemm_launch_pair(p, &g, bn, grid, /*fused=*/true, cs);
  } else {
    if (dynamic_sched()) p.sched = args->counters + SYN_MAX_WAVES + SYN_MAX_COMM_OPS;
    grid = std::min(grid, p.total_tiles);
    if (grid <= 0) return SYN_ERR_INVALID;
    rc = gemm_launch(p, bn, /*fused=*/true, grid, cs);
  }
  if (rc != SYN_OK || !args->reduce_pass) return rc;
  // ---- reduce pass: one launch per row piece of the own slab, its flag raised behind it
  int sms = 0;
  rc = device_sm_count(&sms);
  if (rc != SYN_OK) return rc;
  for (size_t gi = 0; gi < groups.size(); ++gi) {
    RsReduceParams q;
    memset(&q, 0, sizeof(q));
    q.out = static_cast<char*>(args->out) + static_cast<size_t>(groups[gi].off) * ldo * 2;
    q.ldo = ldo;
    q.rows = groups[gi].rows;
    q.n_vec = g.N / 8;
    q.num_red = n_red;
    q.dtype = p.dtype;
    for (int i = 0; i < n_red; ++i) {
      q.src[i] = static_cast<const char*>(p.red_src[i]) + static_cast<size_t>(groups[gi].off) * g.N * 2;
      q.sig[i] = static_cast<int16_t>(groups[gi].sig[i]);
    }
    q.src_ld = g.N;
    q.flags = p.red_flags;
    q.value = epoch;
    q.timeout_ns = p.timeout_ns;
    q.status = p.status;
    q.wave = static_cast<int>(gi);
    const size_t total = static_cast<size_t>(q.rows) * q.n_vec;
    const int blocks = static_cast<int>(std::min<size_t>((total + 255) / 256, static_cast<size_t>(sms) * 4));
    rs_reduce_kernel<<<blocks, 256, 0, cs>>>(q);
    SYN_CUDA_TRY(cudaGetLastError());
    if (args->out_flags != nullptr) {
      rc = syn_flag_set(args->out_flags + gi, epoch, stream);
      if (rc != SYN_OK) return rc;
    }
  }
  return SYN_OK;
}

}  // extern "C"
