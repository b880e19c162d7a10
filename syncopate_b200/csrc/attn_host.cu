// Host side of syn_attention: argument checks, tensor maps, wave table, comm-op table, launch.
#include "attn_sm100.cuh"
#include "host_util.h"

namespace syn {

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

static int check_strides(const int64_t s[3]) {
  for (int i = 0; i < 3; ++i)
    if (s[i] < 0 || (s[i] % 8) != 0) return SYN_ERR_INVALID;
  return SYN_OK;
}

template <bool FUSED>
static int launch_attn(const AttnParams& p, int grid, cudaStream_t stream) {
  constexpr int smem = 1024 + (2 + 2 * ATTN_KV_STAGES) * ATTN_TILE_BYTES + (FUSED ? COMM_NBUF * COMM_PIECE : 0) + 512;
  static_assert(smem <= 232448, "attention kernel exceeds the shared memory of an SM");
  auto kern = attn_kernel<FUSED>;
  static int configured_dev = -1;
  int dev = 0;
  SYN_CUDA_TRY(cudaGetDevice(&dev));
  if (configured_dev != dev) {
    SYN_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured_dev = dev;
  }
  kern<<<grid, 256, smem, stream>>>(p);
  SYN_CUDA_TRY(cudaGetLastError());
  return SYN_OK;
}

}  // namespace syn

extern "C" int syn_attention(const syn_attn_args* a, const syn_schedule* sched, const syn_attn_comm* comm,
                             void* stream) {
  using namespace syn;
  if (a == nullptr || sched == nullptr) return SYN_ERR_INVALID;
  if (a->q == nullptr || a->k == nullptr || a->v == nullptr || a->o == nullptr || a->lse == nullptr ||
      a->visit == nullptr)
    return SYN_ERR_INVALID;
  if (a->D != ATTN_D) return SYN_ERR_UNSUPPORTED;
  if (a->dtype != SYN_DTYPE_F16 && a->dtype != SYN_DTYPE_BF16) return SYN_ERR_UNSUPPORTED;
  if (a->Z <= 0 || a->Hq <= 0 || a->Hkv <= 0 || a->Sq <= 0 || a->Skv <= 0) return SYN_ERR_INVALID;
  if (a->Hq % a->Hkv != 0) return SYN_ERR_INVALID;
  if (a->epoch <= 0) return SYN_ERR_INVALID;
  if (!aligned16(a->q) || !aligned16(a->k) || !aligned16(a->v) || !aligned16(a->o)) return SYN_ERR_INVALID;
  if (check_strides(a->q_strides) || check_strides(a->k_strides) || check_strides(a->v_strides) ||
      check_strides(a->o_strides))
    return SYN_ERR_INVALID;
  if (sched->ndim != 4 || sched->num_waves <= 0 || sched->offsets == nullptr || sched->shapes == nullptr)
    return SYN_ERR_INVALID;
  if (sched->num_waves > ATTN_MAX_WAVES) return SYN_ERR_TOO_LARGE;

  AttnParams p;
  memset(&p, 0, sizeof(p));
  int rc = encode_tmap_4d_sw128(&p.tmap_q, a->q, a->Z, a->Hq, a->Sq, ATTN_D, a->q_strides[0], a->q_strides[1],
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
  p.Z = a->Z;
  p.Hq = a->Hq;
  p.Hkv = a->Hkv;
  p.Sq = a->Sq;
  p.Skv = a->Skv;
  p.q_tiles = (a->Sq + ATTN_BM - 1) / ATTN_BM;
  p.causal = a->causal ? 1 : 0;
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

  int sms = 0;
  rc = device_sm_count(&sms);
  if (rc != SYN_OK) return rc;
  const int grid = a->num_sms > 0 ? (a->num_sms < sms ? a->num_sms : sms) : sms;
  const long pairs = static_cast<long>(a->Z) * a->Hq * ((p.q_tiles + 1) / 2);
  p.own_pairs = (p.causal && pairs >= 2L * grid) ? 1 : 0;
  return fused ? launch_attn<true>(p, grid, static_cast<cudaStream_t>(stream))
               : launch_attn<false>(p, grid, static_cast<cudaStream_t>(stream));
}
