// Host side of the GEMM entry points: argument checks, schedule -> kernel-parameter tables,
// tensor maps, block-size choice, launch.
#include "gemm_host.h"

#include <stdlib.h>

#include <algorithm>

#include "gemm2_sm100.cuh"

namespace syn {

static inline int cdiv(int a, int b) { return (a + b - 1) / b; }

static const int kBlockN[] = {256, 224, 192, 160, 128, 96, 64};

static bool block_n_ok(const syn_schedule* s, int N, int bn) {
  if (s == nullptr) return true;
  for (int w = 0; w < s->num_waves; ++w) {
    const int off = s->offsets[w * 2 + 1], len = s->shapes[w * 2 + 1];
    if (off % bn != 0) return false;
    if (len % bn != 0 && off + len != N) return false;
  }
  return true;
}

static long count_tiles(const syn_schedule* s, int M, int N, int bn) {
  if (s == nullptr) return static_cast<long>(cdiv(M, GEMM_BM)) * cdiv(N, bn);
  long t = 0;
  for (int w = 0; w < s->num_waves; ++w)
    t += static_cast<long>(cdiv(s->shapes[w * 2], GEMM_BM)) * cdiv(s->shapes[w * 2 + 1], bn);
  return t;
}

// Time of one 64-deep k-block of a tile, in ns, measured on B200 with M = 8192, K = 8192 under load
// (one-CTA kernel / CTA-pair kernel).  Narrow tiles pay a fixed cost per MMA; the one-CTA kernel
// at BN = 256 is limited by shared-memory operand traffic, which the pair form halves for B.
static double kblock_ns(int bn, bool pair) {
  switch (bn) {
    case 256: return pair ? 385.0 : 427.0;
    case 224: return 390.0;
    case 192: return 344.0;
    case 160: return 328.0;
    case 128: return 320.0;
    case 96: return 300.0;
    default: return 290.0;
  }
}

static bool pair_shape_ok(const syn_schedule* s, int M) {
  if (s == nullptr) return M % 256 == 0;
  for (int w = 0; w < s->num_waves; ++w)
    if ((s->offsets[w * 2] % 256) || (s->shapes[w * 2] % 256)) return false;
  return true;
}

// Chooses the tile width (and whether the CTA-pair kernel is used, when `pair_out` is given)
// with the fewest persistent rounds weighted by the measured k-block time.
int pick_block_n(const syn_schedule* s, int M, int N, int num_sms, int multiple, bool* pair_out) {
  int best = 0;
  bool best_pair = false;
  double best_cost = 0;
  const bool may_pair = pair_out != nullptr && num_sms >= 2 && pair_shape_ok(s, M);
  for (int use_pair = 0; use_pair <= (may_pair ? 1 : 0); ++use_pair) {
    for (int bn : kBlockN) {
      if (bn % multiple != 0) continue;
      if (!block_n_ok(s, N, bn)) continue;
      long tiles = count_tiles(s, M, N, bn);
      long units = num_sms;
      if (use_pair) {
        tiles = (tiles + 1) / 2;  // 256-row tiles
        units = num_sms / 2;
      }
      const long rounds = (tiles + units - 1) / units;
      const double cost = static_cast<double>(rounds) * kblock_ns(bn, use_pair != 0);
      if (best == 0 || cost < best_cost - 1e-9) {
        best = bn;
        best_pair = use_pair != 0;
        best_cost = cost;
      }
    }
  }
  if (pair_out != nullptr) *pair_out = best_pair;
  return best;
}

int validate_schedule_2d(const syn_schedule* s, int M, int N, int bn) {
  if (s == nullptr) return SYN_OK;
  if (s->ndim != 2 || s->num_waves <= 0 || s->offsets == nullptr || s->shapes == nullptr) return SYN_ERR_INVALID;
  if (s->num_waves > GEMM_MAX_WAVES) return SYN_ERR_TOO_LARGE;
  for (int w = 0; w < s->num_waves; ++w) {
    const int om = s->offsets[w * 2], on = s->offsets[w * 2 + 1];
    const int sm = s->shapes[w * 2], sn = s->shapes[w * 2 + 1];
    if (om < 0 || on < 0 || sm <= 0 || sn <= 0) return SYN_ERR_SHAPE;
    if (om + sm > M || on + sn > N) return SYN_ERR_SHAPE;
    if (om % GEMM_BM != 0 || on % bn != 0) return SYN_ERR_SHAPE;
    if (sm % GEMM_BM != 0 && om + sm != M) return SYN_ERR_SHAPE;
    if (sn % bn != 0 && on + sn != N) return SYN_ERR_SHAPE;
  }
  return SYN_OK;
}

int gemm_fill_common(GemmParams* p, const syn_gemm_args* a, const syn_schedule* sched, int bn) {
  if (a == nullptr || a->a == nullptr || a->b == nullptr || a->c == nullptr) return SYN_ERR_INVALID;
  if (a->M <= 0 || a->N <= 0 || a->K <= 0) return SYN_ERR_INVALID;
  if (a->dtype != SYN_DTYPE_F16 && a->dtype != SYN_DTYPE_BF16) return SYN_ERR_UNSUPPORTED;
  if (a->block_m != 0 && a->block_m != GEMM_BM) return SYN_ERR_UNSUPPORTED;
  if (a->block_k != 0 && a->block_k != GEMM_BK) return SYN_ERR_UNSUPPORTED;
  const int lda = a->lda ? a->lda : a->K, ldb = a->ldb ? a->ldb : a->K, ldc = a->ldc ? a->ldc : a->N;
  if (lda < a->K || ldb < a->K || ldc < a->N) return SYN_ERR_INVALID;
  // TMA wants 16-byte aligned bases and row pitches; the epilogue stores 16-byte vectors
  if ((lda % 8) || (ldb % 8) || (ldc % 8) || (a->N % 8)) return SYN_ERR_INVALID;
  if ((reinterpret_cast<uintptr_t>(a->a) & 15) || (reinterpret_cast<uintptr_t>(a->b) & 15) ||
      (reinterpret_cast<uintptr_t>(a->c) & 15))
    return SYN_ERR_INVALID;
  int rc = validate_schedule_2d(sched, a->M, a->N, bn);
  if (rc != SYN_OK) return rc;

  memset(p, 0, sizeof(*p));
  for (int i = 0; i < GEMM_MAX_WAVES; ++i) p->routes[i].tmap = -1;  // direct stores unless a caller says otherwise
  rc = encode_tmap_2d_sw128(&p->tmap_a, a->a, a->M, a->K, lda, GEMM_BM, GEMM_BK);
  if (rc != SYN_OK) return rc;
  rc = encode_tmap_2d_sw128(&p->tmap_b, a->b, a->N, a->K, ldb, bn, GEMM_BK);
  if (rc != SYN_OK) return rc;
  p->c = a->c;
  p->ldc = ldc;
  p->M = a->M;
  p->N = a->N;
  p->K = a->K;
  p->k_blocks = cdiv(a->K, GEMM_BK);
  p->dtype = a->dtype;
  p->idesc = make_idesc_f16(GEMM_BM, bn, a->dtype == SYN_DTYPE_BF16 ? 1u : 0u, 0, 0);
  p->group_m = a->group_size_m > 0 ? a->group_size_m : 8;
  p->csig = a->consumer_signal_ptr;
  p->counters = a->producer_counter_ptr;
  p->signal_value = a->signal_value ? a->signal_value : 1;
  p->timeout_ns = a->timeout_ns ? a->timeout_ns : 2000000000ull;
  p->status = a->status;
  p->sched = a->sched_counter;
  p->trace = reinterpret_cast<unsigned long long*>(a->trace);

  int cum = 0;
  if (sched == nullptr) {
    GemmWave& w = p->waves[0];
    w.tiles_m = static_cast<int16_t>(cdiv(a->M, GEMM_BM));
    w.tiles_n = static_cast<int16_t>(cdiv(a->N, bn));
    w.off_m = w.off_n = 0;
    w.csig = -1;
    w.route = -1;
    cum = w.tiles_m * w.tiles_n;
    w.cum = cum;
    p->num_waves = 1;
  } else {
    for (int i = 0; i < sched->num_waves; ++i) {
      GemmWave& w = p->waves[i];
      const int tm = cdiv(sched->shapes[i * 2], GEMM_BM), tn = cdiv(sched->shapes[i * 2 + 1], bn);
      if (tm > 32767 || tn > 32767) return SYN_ERR_TOO_LARGE;
      w.tiles_m = static_cast<int16_t>(tm);
      w.tiles_n = static_cast<int16_t>(tn);
      w.off_m = static_cast<int16_t>(sched->offsets[i * 2] / GEMM_BM);
      w.off_n = static_cast<int16_t>(sched->offsets[i * 2 + 1] / bn);
      const int sig = sched->signals ? sched->signals[i] : -1;
      if (sig > 32767) return SYN_ERR_TOO_LARGE;
      w.csig = static_cast<int16_t>(a->consumer_signal_ptr != nullptr ? sig : -1);
      w.route = -1;
      cum += tm * tn;
      w.cum = cum;
    }
    p->num_waves = sched->num_waves;
  }
  p->total_tiles = cum;
  return SYN_OK;
}

// `configure_only`: load the kernel and set its shared-memory limit, launch nothing.
template <int BN, bool FUSED>
static int launch_bn(const GemmParams& p, int grid, cudaStream_t stream, bool configure_only = false) {
  using L = GemmSmem<BN>;
  constexpr int kMaxSmem = 232448;
  constexpr int kFixed = 1024 /*alignment slack*/ + (FUSED ? COMM_NBUF * COMM_PIECE : 0) + 512 /*barriers, queues*/;
  constexpr int kStagesRaw = (kMaxSmem - kFixed) / L::STAGE_BYTES;
  constexpr int STAGES = kStagesRaw > 6 ? 6 : kStagesRaw;
  static_assert(STAGES >= 3, "shared-memory ring too shallow");
  constexpr int smem = STAGES * L::STAGE_BYTES + kFixed;
  auto kern = gemm_kernel<BN, STAGES, FUSED>;
  static bool configured = false;  // per instantiation; attribute is per device but all devices are B200s
  static int configured_dev = -1;
  int dev = 0;
  SYN_CUDA_TRY(cudaGetDevice(&dev));
  if (!configured || configured_dev != dev) {
    SYN_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured = true;
    configured_dev = dev;
  }
  if (configure_only) return SYN_OK;
  kern<<<grid, GEMM_THREADS, smem, stream>>>(p);
  SYN_CUDA_TRY(cudaGetLastError());
  return SYN_OK;
}

template <int BN, bool FUSED>
static int launch_pair_bn(const GemmParams& p, const CUtensorMap& tmap_b_half, int pair_tiles, int grid,
                          const PairTail& tail, cudaStream_t stream, bool configure_only = false) {
  constexpr int kStage = GEMM_BM * GEMM_BK * 2 + (BN / 2) * GEMM_BK * 2;
  constexpr int kFixed = 1024 + 512 + (FUSED ? COMM_NBUF * COMM_PIECE : 0);
  constexpr int kStagesRaw = (232448 - kFixed) / kStage;
  constexpr int STAGES = kStagesRaw > 8 ? 8 : kStagesRaw;
  static_assert(STAGES >= 3, "shared-memory ring too shallow");
  constexpr int smem = STAGES * kStage + kFixed;
  auto kern = gemm2_kernel<BN, STAGES, FUSED>;
  static int configured_dev = -1;
  int dev = 0;
  SYN_CUDA_TRY(cudaGetDevice(&dev));
  if (configured_dev != dev) {
    SYN_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured_dev = dev;
  }
  if (configure_only) return SYN_OK;
  kern<<<grid, GEMM_THREADS, smem, stream>>>(p, tmap_b_half, pair_tiles, tail);
  SYN_CUDA_TRY(cudaGetLastError());
  return SYN_OK;
}

// CTA-pair kernel: 256-row tiles.  Usable when every wave starts and ends on a 256-row boundary and
// tiles are handed out round-robin (no grid-wide tile counter).  SYNCOPATE_B200_NO_PAIR=1 keeps the
// one-CTA kernel (tuning aid).
bool pair_eligible(const GemmParams& p, int bn, int grid) {
  static int disabled = -1;
  if (disabled < 0) {
    const char* e = getenv("SYNCOPATE_B200_NO_PAIR");
    disabled = (e != nullptr && e[0] == '1') ? 1 : 0;
  }
  if (disabled || grid < 2 || p.sched != nullptr) return false;
  if (bn % 32 != 0 || bn < 64) return false;
  for (int w = 0; w < p.num_waves; ++w) {
    if ((p.waves[w].tiles_m & 1) || (p.waves[w].off_m & 1)) return false;
    if (p.waves[w].route >= 0 && p.routes[p.waves[w].route].tmap >= 0 && bn % 64 != 0) return false;
  }
  return true;
}

int gemm_launch_pair(const GemmParams& p_in, const syn_gemm_args* a, int bn, int grid, bool fused,
                     cudaStream_t stream) {
  GemmParams p = p_in;
  p.idesc = make_idesc_f16(GEMM2_BM, bn, a->dtype == SYN_DTYPE_BF16 ? 1u : 0u, 0, 0);
  CUtensorMap tmap_b_half;
  const int ldb = a->ldb ? a->ldb : a->K;
  int rc = encode_tmap_2d_sw128(&tmap_b_half, a->b, a->N, a->K, ldb, bn / 2, GEMM_BK);
  if (rc != SYN_OK) return rc;
  int pair_tiles = 0;
  bool routed = false;
  for (int w = 0; w < p.num_waves; ++w) {
    pair_tiles += (p.waves[w].tiles_m >> 1) * p.waves[w].tiles_n;
    routed = routed || p.waves[w].route >= 0;
  }
  int g = std::min(grid & ~1, 2 * pair_tiles);
  if (g < 2) return SYN_ERR_INVALID;
  // Tail splitting: a small remainder after the last full round is cut along K over all pairs
  // instead of occupying a round of its own.  Needs the caller's zeroed workspace, and plain local
  // stores (a routed tile is counted, staged or reduced where it is finished).
  PairTail tail;
  memset(&tail, 0, sizeof(tail));
  const int pairs = g / 2;
  const int rem = pair_tiles % pairs, rounds = pair_tiles / pairs;
  if (!routed && p.num_kgates == 0 && a->workspace != nullptr && rounds >= 1 && rem > 0 && rem * 4 <= pairs) {
    const int slices = std::min(std::min(pairs / rem, p.k_blocks), 32);
    const size_t need = 256 + static_cast<size_t>(rem) * slices * GEMM2_BM * bn * sizeof(float);
    if (slices >= 2 && a->workspace_bytes >= need && (reinterpret_cast<uintptr_t>(a->workspace) & 255) == 0) {
      tail.tiles = rem;
      tail.slices = slices;
      tail.first_tile = rounds * pairs;
      tail.count = static_cast<unsigned int*>(a->workspace);
      tail.ws = reinterpret_cast<float*>(static_cast<char*>(a->workspace) + 256);
    }
  }
#define SYN_PAIR_CASE(BN_)                                                                         \
  case BN_:                                                                                        \
    return fused ? launch_pair_bn<BN_, true>(p, tmap_b_half, pair_tiles, g, tail, stream)           \
                 : launch_pair_bn<BN_, false>(p, tmap_b_half, pair_tiles, g, tail, stream);
  switch (bn) {
    SYN_PAIR_CASE(256)
    SYN_PAIR_CASE(224)
    SYN_PAIR_CASE(192)
    SYN_PAIR_CASE(160)
    SYN_PAIR_CASE(128)
    SYN_PAIR_CASE(96)
    SYN_PAIR_CASE(64)
    default:
      return SYN_ERR_UNSUPPORTED;
  }
#undef SYN_PAIR_CASE
}

int gemm_launch(const GemmParams& p, int bn, bool fused, int grid, cudaStream_t stream) {
#define SYN_BN_CASE(BN_)                                                     \
  case BN_:                                                                  \
    return fused ? launch_bn<BN_, true>(p, grid, stream) : launch_bn<BN_, false>(p, grid, stream);
  switch (bn) {
    SYN_BN_CASE(256)
    SYN_BN_CASE(224)
    SYN_BN_CASE(192)
    SYN_BN_CASE(160)
    SYN_BN_CASE(128)
    SYN_BN_CASE(96)
    SYN_BN_CASE(64)
    default:
      return SYN_ERR_UNSUPPORTED;
  }
#undef SYN_BN_CASE
}

int preload_gemm_kernels() {
  static GemmParams p;  // never read: configure_only
  static CUtensorMap map;
  static PairTail tail;
  int rc = SYN_OK;
#define SYN_PRELOAD(BN_)                                                              \
  if (rc == SYN_OK) rc = launch_bn<BN_, false>(p, 0, nullptr, true);                  \
  if (rc == SYN_OK) rc = launch_bn<BN_, true>(p, 0, nullptr, true);                   \
  if (rc == SYN_OK) rc = launch_pair_bn<BN_, false>(p, map, 0, 0, tail, nullptr, true); \
  if (rc == SYN_OK) rc = launch_pair_bn<BN_, true>(p, map, 0, 0, tail, nullptr, true);
  SYN_PRELOAD(256)
  SYN_PRELOAD(224)
  SYN_PRELOAD(192)
  SYN_PRELOAD(160)
  SYN_PRELOAD(128)
  SYN_PRELOAD(96)
  SYN_PRELOAD(64)
#undef SYN_PRELOAD
  return rc;
}

int gemm_resolve_grid_and_bn(const syn_gemm_args* a, const syn_schedule* sched, int* grid, int* bn, int multiple,
                             bool* pair_out) {
  int sms = 0;
  int rc = device_sm_count(&sms);
  if (rc != SYN_OK) return rc;
  int g = a->num_sms > 0 ? std::min(a->num_sms, sms) : sms;
  int b = a->block_n;
  if (pair_out != nullptr) *pair_out = true;  // an explicit tile width leaves the kernel choice to eligibility
  if (b == 0) b = pick_block_n(sched, a->M, a->N, g, multiple, pair_out);
  if (b == 0 || b % multiple != 0) return SYN_ERR_SHAPE;
  *grid = g;
  *bn = b;
  return SYN_OK;
}

// A consumer schedule over (M, N, K): every wave covers all of C and one range of K (A arrives as
// column ranges, e.g. behind an all-to-all that splits the contraction axis).  The ranges become
// the kernel's K gates, in wave (= arrival) order.
int fill_kgates(GemmParams* p, const syn_gemm_args* a, const syn_schedule* s) {
  if (s->num_waves <= 0 || s->offsets == nullptr || s->shapes == nullptr) return SYN_ERR_INVALID;
  if (s->num_waves > GEMM_MAX_KGATES) return SYN_ERR_TOO_LARGE;
  long covered = 0;
  for (int w = 0; w < s->num_waves; ++w) {
    const int32_t* off = s->offsets + 3 * w;
    const int32_t* shp = s->shapes + 3 * w;
    if (off[0] != 0 || off[1] != 0 || shp[0] != a->M || shp[1] != a->N) return SYN_ERR_UNSUPPORTED;
    if (off[2] < 0 || shp[2] <= 0 || off[2] + shp[2] > a->K) return SYN_ERR_SHAPE;
    if (off[2] % GEMM_BK != 0) return SYN_ERR_SHAPE;
    if (shp[2] % GEMM_BK != 0 && off[2] + shp[2] != a->K) return SYN_ERR_SHAPE;
    for (int v = 0; v < w; ++v) {  // ranges must not overlap
      const int o2 = s->offsets[3 * v + 2], n2 = s->shapes[3 * v + 2];
      if (off[2] < o2 + n2 && o2 < off[2] + shp[2]) return SYN_ERR_SHAPE;
    }
    const int sig = s->signals ? s->signals[w] : -1;
    if (sig > 32767) return SYN_ERR_TOO_LARGE;
    p->kgate_kb0[w] = static_cast<int16_t>(off[2] / GEMM_BK);
    p->kgate_kb1[w] = static_cast<int16_t>((off[2] + shp[2] + GEMM_BK - 1) / GEMM_BK);
    p->kgate_sig[w] = static_cast<int16_t>(a->consumer_signal_ptr != nullptr ? sig : -1);
    covered += shp[2];
  }
  if (covered != a->K) return SYN_ERR_SHAPE;
  p->num_kgates = s->num_waves;
  return SYN_OK;
}

}  // namespace syn

extern "C" {

int syn_gemm_mod1d(const syn_gemm_args* args, int num_waves, int stride, int starting_offset, int axis, void* stream) {
  // closed form -> wave table: block w starts at (starting_offset + w * stride) mod (stride * num_waves)
  // along `axis`, spans the other axis, and waits for flag w - 1 (the first block is resident)
  if (args == nullptr || num_waves <= 0 || num_waves > SYN_MAX_WAVES || stride <= 0 || starting_offset < 0) return SYN_ERR_INVALID;
  if (axis != 0 && axis != 1) return SYN_ERR_UNSUPPORTED;
  const long extent = static_cast<long>(stride) * num_waves;
  if (extent != (axis == 0 ? args->M : args->N) || starting_offset % stride != 0 || starting_offset >= extent) return SYN_ERR_SHAPE;
  int32_t offs[2 * SYN_MAX_WAVES], shapes[2 * SYN_MAX_WAVES], sigs[SYN_MAX_WAVES];
  for (int w = 0; w < num_waves; ++w) {
    const int at = static_cast<int>((starting_offset + static_cast<long>(w) * stride) % extent);
    offs[2 * w + axis] = at;
    offs[2 * w + 1 - axis] = 0;
    shapes[2 * w + axis] = stride;
    shapes[2 * w + 1 - axis] = axis == 0 ? args->N : args->M;
    sigs[w] = w - 1;
  }
  syn_schedule s;
  memset(&s, 0, sizeof(s));
  s.num_waves = num_waves;
  s.ndim = 2;
  s.offsets = offs;
  s.shapes = shapes;
  s.signals = sigs;
  return syn_gemm(args, &s, nullptr, stream);
}

int syn_gemm_pick_block_n(int M, int N, int num_sms) {
  if (M <= 0 || N <= 0 || num_sms <= 0) return SYN_ERR_INVALID;
  return syn::pick_block_n(nullptr, M, N, num_sms, 32, nullptr);
}

int syn_gemm(const syn_gemm_args* args, const syn_schedule* sched, const syn_schedule* producer_sched,
             void* stream) {
  using namespace syn;
  if (args == nullptr) return SYN_ERR_INVALID;
  // a consumer schedule over (M, N, K) gates ranges of K; the tiles then walk C as one wave
  const syn_schedule* kgates = (sched != nullptr && sched->ndim == 3) ? sched : nullptr;
  if (kgates != nullptr) {
    if (producer_sched != nullptr) return SYN_ERR_UNSUPPORTED;
    sched = nullptr;
  }
  int grid = 0, bn = 0;
  bool want_pair = false;
  int rc = gemm_resolve_grid_and_bn(args, sched ? sched : producer_sched, &grid, &bn, 32,
                                    args->sched_counter == nullptr ? &want_pair : nullptr);
  if (rc != SYN_OK) return rc;
  const syn_schedule* order = sched ? sched : producer_sched;
  GemmParams p;
  rc = gemm_fill_common(&p, args, order, bn);
  if (rc != SYN_OK) return rc;
  if (kgates != nullptr) {
    rc = fill_kgates(&p, args, kgates);
    if (rc != SYN_OK) return rc;
  }
  bool fused = false;
  if (producer_sched != nullptr && args->producer_signal_ptr != nullptr) {
    if (args->producer_counter_ptr == nullptr) return SYN_ERR_INVALID;
    if (sched != nullptr) {
      // dual role: both schedules must walk the same tiles in the same order
      if (sched->num_waves != producer_sched->num_waves) return SYN_ERR_SHAPE;
      for (int i = 0; i < sched->num_waves * 2; ++i)
        if (sched->offsets[i] != producer_sched->offsets[i] || sched->shapes[i] != producer_sched->shapes[i])
          return SYN_ERR_SHAPE;
    }
    rc = validate_schedule_2d(producer_sched, args->M, args->N, bn);
    if (rc != SYN_OK) return rc;
    for (int i = 0; i < producer_sched->num_waves; ++i) {
      const int sig = producer_sched->signals ? producer_sched->signals[i] : -1;
      if (sig < 0) continue;
      GemmRoute& r = p.routes[i];
      r.base = static_cast<char*>(args->c) +
               static_cast<size_t>(producer_sched->offsets[i * 2]) * p.ldc * 2;
      r.ld = p.ldc;
      r.flag = args->producer_signal_ptr + sig;
      r.gate = nullptr;
      r.reduce = 0;
      p.waves[i].route = static_cast<int16_t>(i);
      fused = true;
    }
  }
  if (want_pair && pair_eligible(p, bn, grid))
    return gemm_launch_pair(p, args, bn, grid, fused, static_cast<cudaStream_t>(stream));
  grid = std::min(grid, p.total_tiles);
  if (grid <= 0) return SYN_ERR_INVALID;
  return gemm_launch(p, bn, fused, grid, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
