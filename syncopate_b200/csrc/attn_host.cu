// Host side of syn_attention: argument checks, tensor maps, wave table, comm-op table, launch.
#include "attn2_sm100.cuh"
#include "host_util.h"

#include <algorithm>
#include <mutex>
#include <vector>

namespace syn {

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

static int check_strides(const int64_t s[3]) {
  for (int i = 0; i < 3; ++i)
    if (s[i] < 0 || (s[i] % 8) != 0) return SYN_ERR_INVALID;
  return SYN_OK;
}

template <bool FUSED, bool BF16>
static int launch_attn(const AttnParams& p, int grid, cudaStream_t stream, bool configure_only = false) {
  constexpr int smem = 1024 + (2 + 2 * ATTN_KV_STAGES) * ATTN_TILE_BYTES + (FUSED ? COMM_NBUF * COMM_PIECE : 0) + 512;
  static_assert(smem <= 232448, "attention kernel exceeds the shared memory of an SM");
  auto kern = attn_kernel<FUSED, BF16>;
  static int configured_dev = -1;
  int dev = 0;
  SYN_CUDA_TRY(cudaGetDevice(&dev));
  if (configured_dev != dev) {
    SYN_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured_dev = dev;
  }
  if (configure_only) return SYN_OK;
  kern<<<grid, 256, smem, stream>>>(p);
  SYN_CUDA_TRY(cudaGetLastError());
  return SYN_OK;
}

template <bool FUSED, bool BF16>
static int launch_attn2(const AttnParams& p, int grid, cudaStream_t stream, bool configure_only = false) {
  constexpr int smem = 1024 + (2 + 2 * ATTN_KV_STAGES) * ATTN_TILE_BYTES + (FUSED ? COMM_NBUF * COMM_PIECE : 0) + 512;
  static_assert(smem <= 232448, "attention kernel exceeds the shared memory of an SM");
  auto kern = attn2_kernel<FUSED, BF16>;
  static int configured_dev = -1;
  int dev = 0;
  SYN_CUDA_TRY(cudaGetDevice(&dev));
  if (configured_dev != dev) {
    SYN_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured_dev = dev;
  }
  if (configure_only) return SYN_OK;
  kern<<<grid, ATTN2_THREADS, smem, stream>>>(p);
  SYN_CUDA_TRY(cudaGetLastError());
  return SYN_OK;
}

int preload_attn_kernels() {
  static AttnParams p;  // never read: configure_only
  int rc = launch_attn<false, false>(p, 0, nullptr, true);
  if (rc == SYN_OK) rc = launch_attn<false, true>(p, 0, nullptr, true);
  if (rc == SYN_OK) rc = launch_attn<true, false>(p, 0, nullptr, true);
  if (rc == SYN_OK) rc = launch_attn<true, true>(p, 0, nullptr, true);
  if (rc == SYN_OK) rc = launch_attn2<false, false>(p, 0, nullptr, true);
  if (rc == SYN_OK) rc = launch_attn2<false, true>(p, 0, nullptr, true);
  if (rc == SYN_OK) rc = launch_attn2<true, false>(p, 0, nullptr, true);
  if (rc == SYN_OK) rc = launch_attn2<true, true>(p, 0, nullptr, true);
  return rc;
}

// SYNCOPATE_B200_ATTN_TWO_TILE=0 keeps the one-tile kernel, =2 takes the two-tile kernel whenever
// there are two query tiles (read at every call: test aids).
static int two_tile_mode() {
  const char* e = getenv("SYNCOPATE_B200_ATTN_TWO_TILE");
  if (e != nullptr && e[0] == '0') return 0;
  if (e != nullptr && e[0] == '2') return 2;
  return 1;
}

}  // namespace syn

namespace syn {

// Argument checks and the part of the kernel parameters that both entry points need: shapes,
// flags of the run, the wave table.  Tensor maps, pointers and comm ops are left to the caller.
static int fill_shapes_and_waves(AttnParams& p, const syn_attn_args* a, const syn_schedule* sched) {
  if (a->D != ATTN_D) return SYN_ERR_UNSUPPORTED;
  if (a->dtype != SYN_DTYPE_F16 && a->dtype != SYN_DTYPE_BF16) return SYN_ERR_UNSUPPORTED;
  if (a->Z <= 0 || a->Hq <= 0 || a->Hkv <= 0 || a->Sq <= 0 || a->Skv <= 0) return SYN_ERR_INVALID;
  if (a->Hq % a->Hkv != 0) return SYN_ERR_INVALID;
  if (sched->ndim != 4 || sched->num_waves <= 0 || sched->offsets == nullptr || sched->shapes == nullptr)
    return SYN_ERR_INVALID;
  if (sched->num_waves > ATTN_MAX_WAVES) return SYN_ERR_TOO_LARGE;
  p.Z = a->Z;
  p.Hq = a->Hq;
  p.Hkv = a->Hkv;
  p.Sq = a->Sq;
  p.Skv = a->Skv;
  p.q_tiles = (a->Sq + ATTN_BM - 1) / ATTN_BM;
  p.causal = a->causal ? 1 : 0;
  for (int w = 0; w < sched->num_waves; ++w) {
    const int32_t* off = sched->offsets + 4 * w;
    const int32_t* shp = sched->shapes + 4 * w;
    for (int d = 0; d < 4; ++d)
      if (off[d] < 0 || shp[d] <= 0) return SYN_ERR_SHAPE;
    if (off[0] + shp[0] > a->Z || off[1] + shp[1] > a->Hq || off[2] + shp[2] > a->Sq || off[3] + shp[3] > a->Skv)
      return SYN_ERR_SHAPE;
    if (off[2] % ATTN_BM || off[3] % ATTN_BN || shp[3] % ATTN_BN) return SYN_ERR_SHAPE;
    if (shp[2] % ATTN_BM && off[2] + shp[2] != a->Sq) return SYN_ERR_SHAPE;
    AttnWave& aw = p.waves[w];
    aw.z0 = static_cast<int16_t>(off[0]);
    aw.nz = static_cast<int16_t>(shp[0]);
    aw.h0 = static_cast<int16_t>(off[1]);
    aw.nh = static_cast<int16_t>(shp[1]);
    aw.q0t = off[2] / ATTN_BM;
    aw.nqt = (shp[2] + ATTN_BM - 1) / ATTN_BM;
    aw.kb0 = off[3] / ATTN_BN;
    aw.kb1 = (off[3] + shp[3]) / ATTN_BN;
    aw.sig = (sched->signals && a->signal_ptr) ? sched->signals[w] : -1;
  }
  p.num_waves = sched->num_waves;
  return SYN_OK;
}

static int launch_grid(const syn_attn_args* a, int* grid) {
  int sms = 0;
  int rc = device_sm_count(&sms);
  if (rc != SYN_OK) return rc;
  *grid = a->num_sms > 0 ? (a->num_sms < sms ? a->num_sms : sms) : sms;
  return SYN_OK;
}

// A CTA takes about 1.5 times as long over a key block with two query tiles as with one.  The
// two-tile kernel therefore wins unless the one-tile kernel, spreading the same rows over more
// SMs, needs fewer than 1.5 times as many rounds.
static bool use_two_tile(const AttnParams& p, int grid, bool push = false) {
  const int mode = two_tile_mode();
  if (push) return true;  // the producer role lives in the two-tile kernel
  if (p.q_tiles < 2 || mode == 0) return false;
  if (mode == 2) return true;
  const long heads = static_cast<long>(p.Z) * p.Hq;
  const long rounds_one = (heads * p.q_tiles + grid - 1) / grid;
  const long rounds_two = (heads * ((p.q_tiles + 1) / 2) + grid - 1) / grid;
  return rounds_two * 3 <= rounds_one * 2;
}

// Host twin of the kernels' block_mode: does a 128-row tile starting at qpos0 see key block kb?
static bool block_visible(bool causal, int qpos0, int kpos0) { return !causal || kpos0 <= qpos0 + ATTN_BM - 1; }

}  // namespace syn

extern "C" int syn_attention_plan(const syn_attn_args* a, const syn_schedule* sched, const int32_t* q_pos_host,
                                  const int32_t* kv_pos_host, syn_attn_plan* out) {
  using namespace syn;
  if (a == nullptr || sched == nullptr || out == nullptr) return SYN_ERR_INVALID;
  if ((a->q_pos != nullptr) != (q_pos_host != nullptr) || (a->kv_pos != nullptr) != (kv_pos_host != nullptr))
    return SYN_ERR_INVALID;
  static AttnParams p;  // large; only the shape fields and the wave table are used here
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  memset(&p, 0, sizeof(p));
  int rc = fill_shapes_and_waves(p, a, sched);
  if (rc != SYN_OK) return rc;
  int grid = 0;
  rc = launch_grid(a, &grid);
  if (rc != SYN_OK) {
    // no device to ask (planning ahead on a host without one): trust an explicit CTA count
    if (a->num_sms <= 0) return rc;
    grid = a->num_sms;
  }
  if (grid > SYN_ATTN_PLAN_MAX_GRID) return SYN_ERR_TOO_LARGE;
  const int shift = use_two_tile(p, grid, a->push != nullptr) ? 1 : 0;
  const int per_head = (p.q_tiles + (1 << shift) - 1) >> shift;
  const long n_units = static_cast<long>(p.Z) * p.Hq * per_head;
  if (n_units > SYN_ATTN_PLAN_MAX_UNITS) return SYN_ERR_TOO_LARGE;

  // weight of unit index u of any head inside a wave: key blocks either of its tiles sees, plus a
  // fixed cost for loading Q and writing the result
  std::vector<long> weight(static_cast<size_t>(n_units), 0);
  std::vector<long> w_unit(static_cast<size_t>(per_head));
  std::vector<int> visits(static_cast<size_t>(n_units) * 2, 0);  // waves each tile of a unit takes part in
  std::vector<int> v_unit(static_cast<size_t>(per_head) * 2);
  for (int w = 0; w < p.num_waves; ++w) {
    const AttnWave& aw = p.waves[w];
    for (int u = 0; u < per_head; ++u) {
      long cnt = 0;
      bool tile_seen[2] = {false, false};
      for (int kb = aw.kb0; kb < aw.kb1; ++kb) {
        const int kpos0 = kv_pos_host ? kv_pos_host[kb] : kb * ATTN_BN;
        bool seen = false;
        for (int x = 0; x < (1 << shift); ++x) {
          const int qt = (u << shift) + x;
          if (qt < aw.q0t || qt >= aw.q0t + aw.nqt || qt >= p.q_tiles) continue;
          const int qpos0 = q_pos_host ? q_pos_host[qt] : qt * ATTN_BM;
          const bool vis = block_visible(p.causal != 0, qpos0, kpos0);
          seen = seen || vis;
          tile_seen[x] = tile_seen[x] || vis;
        }
        cnt += seen ? 1 : 0;
      }
      w_unit[u] = cnt > 0 ? cnt + 2 : 0;
      v_unit[2 * u] = tile_seen[0] ? 1 : 0;
      v_unit[2 * u + 1] = tile_seen[1] ? 1 : 0;
    }
    for (int z = aw.z0; z < aw.z0 + aw.nz; ++z)
      for (int h = aw.h0; h < aw.h0 + aw.nh; ++h)
        for (int u = 0; u < per_head; ++u) {
          const size_t id = (static_cast<size_t>(z) * p.Hq + h) * per_head + u;
          weight[id] += w_unit[u];
          visits[2 * id] += v_unit[2 * u];
          visits[2 * id + 1] += v_unit[2 * u + 1];
        }
  }
  // longest first, each to the least loaded CTA
  std::vector<int> order(static_cast<size_t>(n_units));
  for (long i = 0; i < n_units; ++i) order[i] = static_cast<int>(i);
  std::stable_sort(order.begin(), order.end(), [&](int x, int y) { return weight[x] > weight[y]; });
  std::vector<long> load(static_cast<size_t>(grid), 0);
  std::vector<std::vector<uint16_t>> lists(static_cast<size_t>(grid));
  for (int id : order) {
    int best = 0;
    for (int c = 1; c < grid; ++c)
      if (load[c] < load[best]) best = c;
    load[best] += weight[id];
    lists[best].push_back(static_cast<uint16_t>(id));
  }
  memset(out, 0, sizeof(*out));
  out->grid = grid;
  out->unit_rows = ATTN_BM << shift;
  out->num_units = static_cast<int32_t>(n_units);
  int pos = 0;
  for (int c = 0; c < grid; ++c) {
    out->start[c] = static_cast<uint16_t>(pos);
    for (uint16_t id : lists[c]) out->units[pos++] = id;
  }
  for (int c = grid; c <= SYN_ATTN_PLAN_MAX_GRID; ++c) out->start[c] = static_cast<uint16_t>(pos);
  for (long i = 0; i < 2 * n_units; ++i) out->visits[i] = static_cast<uint8_t>(std::min(visits[static_cast<size_t>(i)], 255));
  return SYN_OK;
}

extern "C" int syn_attention(const syn_attn_args* a, const syn_schedule* sched, const syn_attn_comm* comm,
                             void* stream) {
  using namespace syn;
  if (a == nullptr || sched == nullptr) return SYN_ERR_INVALID;
  if (a->q == nullptr || a->k == nullptr || a->v == nullptr || a->o == nullptr || a->lse == nullptr ||
      a->visit == nullptr)
    return SYN_ERR_INVALID;
  if (a->epoch <= 0) return SYN_ERR_INVALID;
  if (!aligned16(a->q) || !aligned16(a->k) || !aligned16(a->v) || !aligned16(a->o)) return SYN_ERR_INVALID;
  if (check_strides(a->q_strides) || check_strides(a->k_strides) || check_strides(a->v_strides) ||
      check_strides(a->o_strides))
    return SYN_ERR_INVALID;

  AttnParams p;
  memset(&p, 0, sizeof(p));
  int rc = fill_shapes_and_waves(p, a, sched);
  if (rc != SYN_OK) return rc;
  rc = encode_tmap_4d_sw128(&p.tmap_q, a->q, a->Z, a->Hq, a->Sq, ATTN_D, a->q_strides[0], a->q_strides[1],
                            a->q_strides[2], ATTN_BM, 64);
  if (rc != SYN_OK) return rc;
  rc = encode_tmap_4d_sw128(&p.tmap_k, a->k, a->Z, a->Hkv, a->Skv, ATTN_D, a->k_strides[0], a->k_strides[1],
                            a->k_strides[2], ATTN_BN, 64);
  if (rc != SYN_OK) return rc;
  rc = encode_tmap_4d_sw128(&p.tmap_v, a->v, a->Z, a->Hkv, a->Skv, ATTN_D, a->v_strides[0], a->v_strides[1],
                            a->v_strides[2], ATTN_BN, 64);
  if (rc != SYN_OK) return rc;
  p.o = a->o;
  p.lse = a->lse;
  p.visit = a->visit;
  p.o_sz = a->o_strides[0];
  p.o_sh = a->o_strides[1];
  p.o_ss = a->o_strides[2];
  p.dtype = a->dtype;
  p.epoch = a->epoch;
  p.scale_log2 = a->sm_scale * 1.4426950408889634f;
  p.q_pos = a->q_pos;
  p.kv_pos = a->kv_pos;
  p.flags = a->signal_ptr;
  p.signal_value = a->signal_value ? a->signal_value : 1;
  p.timeout_ns = a->timeout_ns ? a->timeout_ns : 2000000000ull;
  p.status = a->status;
  const uint32_t fmt = a->dtype == SYN_DTYPE_BF16 ? 1u : 0u;
  p.idesc_qk = make_idesc_f16(ATTN_BM, ATTN_BN, fmt, 0, 0);
  p.idesc_pv = make_idesc_f16(ATTN_BM, ATTN_D, fmt, 0, 1);  // V is read d-contiguous: MN-major B
  bool fused = false;
  if (comm != nullptr && comm->num_ops > 0) {
    if (comm->ops == nullptr || comm->counters == nullptr) return SYN_ERR_INVALID;
    if (comm->num_ops > ATTN_MAX_COMM_OPS) return SYN_ERR_TOO_LARGE;
    if (comm->num_bufs <= 0 || comm->num_bufs > 4) return SYN_ERR_INVALID;
    const int rank = comm->bufs[0].rank, world = comm->bufs[0].world;
    for (int i = 0; i < comm->num_ops; ++i) {
      const syn_copy_op& o = comm->ops[i];
      if (o.src_buf < 0 || o.src_buf >= comm->num_bufs || o.dst_buf < 0 || o.dst_buf >= comm->num_bufs)
        return SYN_ERR_INVALID;
      if (o.src_rank < 0 || o.src_rank >= world || o.dst_rank < 0 || o.dst_rank >= world) return SYN_ERR_INVALID;
      if (o.src_rank != rank && o.dst_rank != rank) return SYN_ERR_INVALID;
      if ((o.src_offset | o.dst_offset | o.src_pitch | o.dst_pitch | o.row_bytes) & 15) return SYN_ERR_INVALID;
      if (o.reduce != 0) return SYN_ERR_UNSUPPORTED;  // comm warps move bytes; reducing copies belong to syn_copy
      CommOp& c = p.comm[i];
      c.src = static_cast<const char*>(comm->bufs[o.src_buf].ptrs[o.src_rank]) + o.src_offset;
      c.dst = static_cast<char*>(comm->bufs[o.dst_buf].ptrs[o.dst_rank]) + o.dst_offset;
      if (c.src == nullptr || c.dst == nullptr) return SYN_ERR_INVALID;
      c.src_pitch = o.src_pitch;
      c.dst_pitch = o.dst_pitch;
      c.rows = o.rows;
      c.row_bytes = o.row_bytes;
      c.wait_flag = nullptr;
      c.set_flag = nullptr;
      if (o.flag >= 0) {
        if (o.flag_rank < 0 || o.flag_rank >= world || comm->flags.ptrs[o.flag_rank] == nullptr) return SYN_ERR_INVALID;
        c.set_flag = static_cast<uint64_t*>(comm->flags.ptrs[o.flag_rank]) + o.flag;
      }
    }
    p.num_comm_ops = comm->num_ops;
    p.counters = comm->counters;
    fused = true;
  }

  int grid = 0;
  rc = launch_grid(a, &grid);
  if (rc != SYN_OK) return rc;
  const bool two = use_two_tile(p, grid, a->push != nullptr);
  if (a->plan != nullptr) {
    const syn_attn_plan& pl = *a->plan;
    const int per_head = two ? (p.q_tiles + 1) / 2 : p.q_tiles;
    if (pl.grid != grid || pl.unit_rows != (two ? 2 * ATTN_BM : ATTN_BM) ||
        pl.num_units != static_cast<long>(a->Z) * a->Hq * per_head || pl.num_units > SYN_ATTN_PLAN_MAX_UNITS)
      return SYN_ERR_INVALID;
    memcpy(p.own_start, pl.start, sizeof(p.own_start));
    memcpy(p.own_units, pl.units, sizeof(p.own_units));
    p.use_lists = 1;
  }
  if (a->push != nullptr) {
    // producer role: destination maps, slab table, per-tile visit counts (from the plan)
    const syn_attn_push& pu = *a->push;
    if (a->plan == nullptr || !two) return SYN_ERR_INVALID;  // needs fixed ownership lists
    if (pu.num_slabs <= 0 || pu.num_slabs > ATTN_MAX_PUSH || pu.slabs == nullptr || pu.counters == nullptr)
      return SYN_ERR_INVALID;
    if (a->Sq % ATTN_BM != 0) return SYN_ERR_SHAPE;
    if (pu.dst.world <= 0 || pu.dst.world > SYN_MAX_WORLD) return SYN_ERR_INVALID;
    for (int c = 0; c < grid; ++c)
      if (a->plan->start[c + 1] - a->plan->start[c] > ATTN_PUSH_MAX_UNITS_PER_CTA) return SYN_ERR_TOO_LARGE;
    memcpy(p.visits, a->plan->visits, sizeof(p.visits));
    int covered = 0;
    for (int i = 0; i < pu.num_slabs; ++i) {
      const syn_attn_push_slab& sl = pu.slabs[i];
      if (sl.q_begin != covered || sl.q_rows <= 0 || (sl.q_begin % ATTN_BM) || (sl.q_rows % ATTN_BM)) return SYN_ERR_SHAPE;
      if (sl.dst_rank < 0 || sl.dst_rank >= pu.dst.world || pu.dst.ptrs[sl.dst_rank] == nullptr) return SYN_ERR_INVALID;
      if (sl.dst_row0 < 0 || sl.dst_row0 + sl.q_rows > pu.dst_rows) return SYN_ERR_SHAPE;
      covered += sl.q_rows;
      AttnPushSlab& ps = p.push[i];
      ps.s0 = sl.q_begin;
      ps.s1 = sl.q_begin + sl.q_rows;
      ps.row0 = sl.dst_row0;
      ps.flag = nullptr;
      if (sl.flag >= 0) {
        if (pu.flags.ptrs[sl.dst_rank] == nullptr) return SYN_ERR_INVALID;
        ps.flag = static_cast<uint64_t*>(pu.flags.ptrs[sl.dst_rank]) + sl.flag;
      }
      // tiles of the slab that any wave visits, over all (z, h)
      int tiles = 0;
      const int per_head = (p.q_tiles + 1) / 2;
      for (long zh = 0; zh < static_cast<long>(a->Z) * a->Hq; ++zh)
        for (int qt = ps.s0 / ATTN_BM; qt < ps.s1 / ATTN_BM; ++qt)
          tiles += p.visits[2 * (zh * per_head + (qt >> 1)) + (qt & 1)] > 0 ? 1 : 0;
      ps.tiles = tiles;
      rc = encode_tmap_4d_sw128(&p.tmap_push[i], pu.dst.ptrs[sl.dst_rank], a->Z, pu.dst_heads, pu.dst_rows, ATTN_D,
                                pu.dst_strides[0], pu.dst_strides[2], pu.dst_strides[1], 32, 64);
      if (rc != SYN_OK) return rc;
    }
    if (covered != a->Sq) return SYN_ERR_SHAPE;
    if (pu.head_offset < 0 || pu.head_offset + a->Hq > pu.dst_heads) return SYN_ERR_SHAPE;
    p.num_push = pu.num_slabs;
    p.push_head0 = pu.head_offset;
    p.push_counters = pu.counters;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (two) {
    // two query tiles per CTA at a time; ownership (and its balanced pairing) is over tile pairs
    const int units = (p.q_tiles + 1) / 2;
    const long pairs = static_cast<long>(a->Z) * a->Hq * ((units + 1) / 2);
    p.own_pairs = (p.causal && pairs >= grid) ? 1 : 0;
    if (a->dtype == SYN_DTYPE_BF16)
      return fused ? launch_attn2<true, true>(p, grid, st) : launch_attn2<false, true>(p, grid, st);
    return fused ? launch_attn2<true, false>(p, grid, st) : launch_attn2<false, false>(p, grid, st);
  }
  const long pairs = static_cast<long>(a->Z) * a->Hq * ((p.q_tiles + 1) / 2);
  p.own_pairs = (p.causal && pairs >= 2L * grid) ? 1 : 0;
  if (a->dtype == SYN_DTYPE_BF16) return fused ? launch_attn<true, true>(p, grid, st) : launch_attn<false, true>(p, grid, st);
  return fused ? launch_attn<true, false>(p, grid, st) : launch_attn<false, false>(p, grid, st);
}
