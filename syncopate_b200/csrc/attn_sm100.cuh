// Flash-attention forward for sm_100a over a wave schedule: tcgen05.mma for S = Q K^T and O += P V,
// S / P / partial O in tensor memory, online softmax in the exp2 domain, causal masking by true
// token positions, grouped-query heads, and log-sum-exp merging of the partial results of a query
// tile that several waves visit.
//
// Follows the behaviour of Syncopate's wave-dispatched FA kernel
// (syncopate/computation/attn/template.py:47-361): a work unit is (z, h, 128-row Q tile) of a wave
// and runs over the wave's KV range (:80-121); a wave with a signal index waits for its flag first
// (:90-97); a Q tile visited again merges (O, log2-LSE) with what is stored (:339-349).  Instead of
// the reference's global spin lock, every Q tile is owned by one CTA for the whole launch (tile
// id modulo grid size), which visits it wave after wave, so merges need no lock.
//
// Roles per CTA (256 threads): warp 0 TMA producer, warp 1 MMA issuer, warp 2 TMEM allocator,
// warp 3 comm warp (copies scheduled chunks between peer-mapped buffers, optional), warps 4-7
// softmax / accumulate / merge / store (thread t owns query row t of the tile).
#pragma once
#include "gemm_sm100.cuh"  // CommOp, comm_warp_run, pack helpers
#include "../../include/syncopate_b200.h"  // plan limits

namespace syn {

constexpr int ATTN_BM = 128;   // query rows per tile
constexpr int ATTN_BN = 128;   // keys per block
constexpr int ATTN_D = 128;    // head dimension
constexpr int ATTN_MAX_WAVES = 96;
constexpr int ATTN_MAX_COMM_OPS = 48;
constexpr int ATTN_KV_STAGES = 2;
constexpr int ATTN_TILE_BYTES = ATTN_BM * ATTN_D * 2;  // 32 KB: two 128 x 64 swizzled boxes

struct AttnWave {
  int16_t z0, nz, h0, nh;  // batch / head box of the wave
  int32_t q0t, nqt;        // first query tile and number of query tiles (units of 128 rows)
  int32_t kb0, kb1;        // key-block range [kb0, kb1) (units of 128 keys)
  int32_t sig;             // flag index to wait for, -1 = none
};

constexpr int ATTN_MAX_PUSH = SYN_MAX_WORLD;
constexpr int ATTN_PUSH_MAX_UNITS_PER_CTA = 64;

// One destination slab of the producer role: query rows [s0, s1) go to one rank's buffer.
struct AttnPushSlab {
  int32_t s0, s1;     // query rows covered
  int32_t row0;       // destination row of s0
  int32_t tiles;      // 128-row tiles (over z and h) whose last visit completes the slab
  uint64_t* flag;     // raised to signal_value once `tiles` tiles have landed; may be null
};

struct AttnParams {
  CUtensorMap tmap_q, tmap_k, tmap_v;  // 4-D (d, s, h, z), box 64 x 128
  void* o;
  float* lse;              // [Z, Hq, Sq] log2 domain
  int32_t* visit;          // [Z, Hq, Sq]: epoch of the last launch that wrote the row
  int64_t o_sz, o_sh, o_ss;  // output strides in elements (z, h, s)
  int32_t Z, Hq, Hkv, Sq, Skv;
  int32_t q_tiles;         // ceil(Sq / 128)
  int32_t causal;
  int32_t own_pairs;       // causal runs with enough tiles: query tiles are owned in balanced pairs
  int32_t dtype;
  int32_t epoch;
  int32_t num_waves;
  int32_t num_comm_ops;
  float scale_log2;        // sm_scale * log2(e)
  const int32_t* q_pos;    // true position of the first row of each query tile, null = tile * 128
  const int32_t* kv_pos;   // true position of the first key of each key block, null = block * 128
  const uint64_t* flags;
  uint32_t* counters;      // comm counters [num_comm_ops]
  uint64_t signal_value;
  uint64_t timeout_ns;
  int32_t* status;
  uint32_t idesc_qk, idesc_pv;
  AttnWave waves[ATTN_MAX_WAVES];
  CommOp comm[ATTN_MAX_COMM_OPS];
  int32_t use_lists;       // 1: ownership comes from the lists below instead of the arithmetic rule
  uint16_t own_start[SYN_ATTN_PLAN_MAX_GRID + 1];
  uint16_t own_units[SYN_ATTN_PLAN_MAX_UNITS];
  // producer role (two-tile kernel): a tile's rows leave for their destination rank at its last visit
  int32_t num_push;        // 0 = off
  int32_t push_head0;      // destination head of head 0
  uint32_t* push_counters; // [num_push] tiles landed per slab, self-resetting
  AttnPushSlab push[ATTN_MAX_PUSH];
  CUtensorMap tmap_push[ATTN_MAX_PUSH];  // 4-D (d, s, h, z) maps of the destination buffers, box 64 x 32
  uint8_t visits[2 * SYN_ATTN_PLAN_MAX_UNITS];  // per (unit, tile): waves it takes part in
};

// Enumerates, in wave order, the units this CTA owns.  All roles run the same enumeration.
// Ownership is fixed for the whole launch.  Non-causal: query tile qt of head (z, h) belongs to CTA
// ((z * Hq + h) * T + qt) mod grid.  Causal: tiles are owned in pairs {j, T-1-j} (tile t has about
// t + 1 visible key blocks, so every pair carries the same work) and pair j of head (z, h)
// belongs to CTA ((z * Hq + h) * ceil(T / 2) + j) mod grid (when the host sets `own_pairs`: enough pairs
// for every CTA).  With `use_lists` the host has planned the ownership instead (syn_attention_plan)
// and the CTA walks its own list of units once per wave.
//
// `shift` = 1 makes the unit a run of two adjacent query tiles (2 * unit, 2 * unit + 1), for the
// kernel that works on two tiles at a time; a wave then touches every such run it overlaps.
struct UnitCursor {
  int wave = 0, zi = 0, hi = 0, slot = -1, half = 0, shift = 0;
  __device__ __forceinline__ bool next(const AttnParams& p, int& z, int& h, int& qtile) {
    const int G = gridDim.x, c = blockIdx.x, T = (p.q_tiles + (1 << shift) - 1) >> shift;
    if (p.use_lists) {
      // planned ownership: walk this CTA's list once per wave (`slot` is the list position)
      const int first = p.own_start[c], last = p.own_start[c + 1];
      if (slot < 0) slot = first;
      while (wave < p.num_waves) {
        const AttnWave& w = p.waves[wave];
        const int lo = w.q0t >> shift, hi = (w.q0t + w.nqt - 1) >> shift;
        while (slot < last) {
          const int id = p.own_units[slot++];
          const int u = id % T, zh = id / T, hh = zh % p.Hq, zz = zh / p.Hq;
          if (u >= lo && u <= hi && hh >= w.h0 && hh < w.h0 + w.nh && zz >= w.z0 && zz < w.z0 + w.nz) {
            z = zz;
            h = hh;
            qtile = u;
            return true;
          }
        }
        slot = first;
        ++wave;
      }
      return false;
    }
    const int slots = p.own_pairs ? (T + 1) / 2 : T;
    while (wave < p.num_waves) {
      const AttnWave& w = p.waves[wave];
      while (zi < w.nz) {
        while (hi < w.nh) {
          const int zz = w.z0 + zi, hh = w.h0 + hi;
          while (true) {
            if (slot < 0) {
              const long base = (static_cast<long>(zz) * p.Hq + hh) * slots;
              slot = static_cast<int>(((c - base) % G + G) % G);  // first slot of this head owned by the CTA
              half = 0;
            } else if (p.own_pairs && half == 0) {
              half = 1;
            } else {
              slot += G;
              half = 0;
            }
            if (slot >= slots) break;
            int qt = slot;
            if (p.own_pairs && half == 1) {
              qt = T - 1 - slot;
              if (qt == slot) continue;  // the middle tile of an odd count is its own partner
            }
            if (qt >= (w.q0t >> shift) && qt <= ((w.q0t + w.nqt - 1) >> shift)) {
              z = zz;
              h = hh;
              qtile = qt;
              return true;
            }
          }
          slot = -1;
          ++hi;
        }
        hi = 0;
        ++zi;
      }
      zi = 0;
      ++wave;
    }
    return false;
  }
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 0 = skip the block (no key visible to any row), 1 = no mask needed, 2 = mask by position.
__device__ __forceinline__ int block_mode(const AttnParams& p, int qpos0, int kb) {
  if (!p.causal) return 1;
  const int kpos0 = p.kv_pos ? __ldg(p.kv_pos + kb) : kb * ATTN_BN;
  if (kpos0 > qpos0 + ATTN_BM - 1) return 0;
  if (kpos0 + ATTN_BN - 1 <= qpos0) return 1;
  return 2;
}

__device__ __forceinline__ uint32_t pack2_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t pack2_f16(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Finalises one query row of a unit: O (fp32, in tensor memory at `o_tmem`, this thread's lane)
// is scaled by 1 / l and stored; if the row was already written in this launch (an earlier wave
// visited it) the stored (O, log2-LSE) and the new ones are merged first
// (syncopate/computation/attn/template.py:339-349).  Every lane of the warp must call it (the
// tensor-memory loads are warp-wide); rows past the end only skip the memory accesses.
//
// With `stage` (shared memory of this warp, 2 x 4 KB: d 0..63 and d 64..127 of its 32 rows in the
// 128-byte swizzle of a TMA store box) the finished row goes there instead of `o`: the caller sends
// it on (producer role).
template <bool BF16>
__device__ __forceinline__ void attn_finish_row(const AttnParams& p, int z, int h, int qt, int row, float m, float l,
                                                uint32_t o_tmem, uint8_t* stage = nullptr) {
  const int srow = qt * ATTN_BM + row;
  const bool valid = srow < p.Sq;
  const size_t stat_idx = (static_cast<size_t>(z) * p.Hq + h) * p.Sq + (valid ? srow : 0);
  uint4* o_ptr = reinterpret_cast<uint4*>(reinterpret_cast<char*>(p.o) +
                                          (z * p.o_sz + h * p.o_sh + static_cast<int64_t>(valid ? srow : 0) * p.o_ss) * 2);
  const bool seen = valid && p.visit[stat_idx] == p.epoch;
  float lse_new = (l > 0.f) ? m + log2f(l) : -INFINITY;
  const float inv_l = (l > 0.f) ? 1.f / l : 0.f;
  float w_new = inv_l, w_old = 0.f;
  if (seen) {
    const float lse_old = p.lse[stat_idx];
    const float mm = fmaxf(lse_old, lse_new);
    if (mm == -INFINITY) {
      w_new = 0.f;
      w_old = 1.f;
    } else {
      const float e_old = exp2f(lse_old - mm), e_new = exp2f(lse_new - mm);
      const float tot = e_old + e_new;
      w_old = e_old / tot;
      w_new = e_new / tot * inv_l;
      lse_new = mm + log2f(tot);
    }
  }
#pragma unroll 1
  for (int v = 0; v < ATTN_D / 32; ++v) {
    uint32_t r[32];
    tmem_ld_32x32(o_tmem + v * 32, r);
    tmem_ld_wait();
    if (valid) {
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) {
        float f[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(r[c4 * 8 + i]) * w_new;
        if (seen) {
          const uint4 old = o_ptr[v * 4 + c4];
          const uint32_t ow[4] = {old.x, old.y, old.z, old.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 t = unpack2(ow[i], p.dtype);
            f[2 * i] += t.x * w_old;
            f[2 * i + 1] += t.y * w_old;
          }
        }
        uint4 out;
        out.x = BF16 ? pack2_bf16(f[0], f[1]) : pack2_f16(f[0], f[1]);
        out.y = BF16 ? pack2_bf16(f[2], f[3]) : pack2_f16(f[2], f[3]);
        out.z = BF16 ? pack2_bf16(f[4], f[5]) : pack2_f16(f[4], f[5]);
        out.w = BF16 ? pack2_bf16(f[6], f[7]) : pack2_f16(f[6], f[7]);
        if (stage != nullptr) {
          // 16-byte chunk v * 4 + c4 of the row's 16: half = chunk / 8, chunk inside the half swizzled
          const int chunk = v * 4 + c4, lane32 = row & 31;
          *reinterpret_cast<uint4*>(stage + (chunk >> 3) * 4096 + lane32 * 128 + (((chunk & 7) ^ (lane32 & 7)) << 4)) = out;
        } else {
          o_ptr[v * 4 + c4] = out;
        }
      }
    }
  }
  if (valid) {
    p.lse[stat_idx] = lse_new;
    p.visit[stat_idx] = p.epoch;
  }
}

template <bool FUSED, bool BF16>
__global__ void __launch_bounds__(256, 1) attn_kernel(const __grid_constant__ AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                                        // 2 tiles
  uint8_t* sK = sQ + 2 * ATTN_TILE_BYTES;                    // ATTN_KV_STAGES tiles
  uint8_t* sV = sK + ATTN_KV_STAGES * ATTN_TILE_BYTES;       // ATTN_KV_STAGES tiles
  uint8_t* ring = sV + ATTN_KV_STAGES * ATTN_TILE_BYTES;     // FUSED only
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring + (FUSED ? COMM_NBUF * COMM_PIECE : 0));
  uint64_t* q_full = bars;            // [2]
  uint64_t* q_empty = bars + 2;       // [2]
  uint64_t* k_full = bars + 4;        // [KV_STAGES]
  uint64_t* k_empty = bars + 6;
  uint64_t* v_full = bars + 8;
  uint64_t* v_empty = bars + 10;
  uint64_t* s_full = bars + 12;       // [2] MMA -> softmax
  uint64_t* p_full = bars + 14;       // [2] softmax -> MMA
  uint64_t* o_full = bars + 16;       // [2] MMA -> softmax
  uint64_t* o_empty = bars + 18;      // [2] softmax -> MMA
  uint64_t* comm_bar = bars + 20;     // [COMM_NBUF]
  uint64_t* done_bar = bars + 20 + COMM_NBUF;  // the issuing warp's products have completed (give-up path)
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 21 + COMM_NBUF);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_holder + 1);
  int* abort_info = const_cast<int*>(abort_word) + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 128);
      mbar_init(&o_full[i], 1);
      mbar_init(&o_empty[i], 128);
    }
    for (int i = 0; i < COMM_NBUF; ++i) mbar_init(&comm_bar[i], 1);
    mbar_init(done_bar, 1);
    *abort_word = 0;
    abort_info[0] = -1;
    abort_info[1] = -1;
    fence_mbar_init();
  }
  if (warp == 2) {
    tmem_alloc(tmem_holder, 512);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tmap(&p.tmap_q);
    prefetch_tmap(&p.tmap_k);
    prefetch_tmap(&p.tmap_v);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const int group = p.Hq / p.Hkv;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      UnitCursor cur;
      int z, h, qt;
      uint32_t u = 0, g = 0;  // running unit / key-block counters (ring positions)
      int flag_wave = -1;     // last wave whose flag this CTA has waited for
      uint32_t kfills = 0, vfills = 0;
      bool ok = true;
      while (ok && cur.next(p, z, h, qt)) {
        if (*abort_word != 0) break;
        const AttnWave& w = p.waves[cur.wave];
        const int qpos0 = p.q_pos ? __ldg(p.q_pos + qt) : qt * ATTN_BM;
        int active = 0;
        for (int kb = w.kb0; kb < w.kb1; ++kb) active += block_mode(p, qpos0, kb) != 0;
        if (active == 0) continue;
        if (cur.wave != flag_wave && w.sig >= 0 && p.flags != nullptr) {
          flag_wave = cur.wave;
          if (!flag_wait_ge(p.flags + w.sig, p.signal_value, abort_word, p.timeout_ns)) {
            if (abort_info[0] < 0) {
              abort_info[0] = cur.wave;
              abort_info[1] = w.sig;
            }
            break;  // the wave's data never arrived: issue no load for it
          }
          fence_proxy_async();
        }
        const int qb = u & 1;
        if (!mbar_wait(&q_empty[qb], ((u >> 1) & 1u) ^ 1u, abort_word, p.timeout_ns)) break;
        mbar_expect_tx(&q_full[qb], ATTN_TILE_BYTES);
        tma_load_4d(sQ + qb * ATTN_TILE_BYTES, &p.tmap_q, &q_full[qb], 0, qt * ATTN_BM, h, z);
        tma_load_4d(sQ + qb * ATTN_TILE_BYTES + ATTN_TILE_BYTES / 2, &p.tmap_q, &q_full[qb], 64, qt * ATTN_BM, h, z);
        ++u;
        const int hk = h / group;
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (block_mode(p, qpos0, kb) == 0) continue;
          const int st = g % ATTN_KV_STAGES;
          const uint32_t par = ((g / ATTN_KV_STAGES) & 1u) ^ 1u;
          if (!mbar_wait(&k_empty[st], par, abort_word, p.timeout_ns)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&k_full[st], ATTN_TILE_BYTES);
          tma_load_4d(sK + st * ATTN_TILE_BYTES, &p.tmap_k, &k_full[st], 0, kb * ATTN_BN, hk, z);
          tma_load_4d(sK + st * ATTN_TILE_BYTES + ATTN_TILE_BYTES / 2, &p.tmap_k, &k_full[st], 64, kb * ATTN_BN, hk, z);
          ++kfills;
          if (!mbar_wait(&v_empty[st], par, abort_word, p.timeout_ns)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&v_full[st], ATTN_TILE_BYTES);
          tma_load_4d(sV + st * ATTN_TILE_BYTES, &p.tmap_v, &v_full[st], 0, kb * ATTN_BN, hk, z);
          tma_load_4d(sV + st * ATTN_TILE_BYTES + ATTN_TILE_BYTES / 2, &p.tmap_v, &v_full[st], 64, kb * ATTN_BN, hk, z);
          ++vfills;
          ++g;
        }
      }
      if (*abort_word != 0) {
        // loads already issued keep writing this CTA's shared memory: wait for them before leaving
        for (int qb = 0; qb < 2; ++qb) drain_stage(&q_full[qb], u / 2 + (static_cast<uint32_t>(qb) < u % 2 ? 1u : 0u), p.timeout_ns);
        for (int st = 0; st < ATTN_KV_STAGES; ++st) {
          drain_stage(&k_full[st], kfills / ATTN_KV_STAGES + (static_cast<uint32_t>(st) < kfills % ATTN_KV_STAGES ? 1u : 0u),
                      p.timeout_ns);
          drain_stage(&v_full[st], vfills / ATTN_KV_STAGES + (static_cast<uint32_t>(st) < vfills % ATTN_KV_STAGES ? 1u : 0u),
                      p.timeout_ns);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // The whole warp walks the units and waits on the barriers; one elected lane issues each
    // tcgen05 instruction, with descriptor words computed as warp-uniform values.
    {
      UnitCursor cur;
      int z, h, qt;
      uint32_t u = 0, g = 0;
      constexpr uint32_t TILE_UNITS = ATTN_TILE_BYTES >> 4;
      const uint32_t desc_hi = static_cast<uint32_t>(make_smem_desc_sw128(0, 16, 1024) >> 32);
      const uint32_t q_lo = static_cast<uint32_t>(make_smem_desc_sw128(smem_u32(sQ), 16, 1024));
      const uint32_t k_lo = static_cast<uint32_t>(make_smem_desc_sw128(smem_u32(sK), 16, 1024));
      const uint32_t v_lo = static_cast<uint32_t>(make_smem_desc_sw128(smem_u32(sV), ATTN_TILE_BYTES / 2, 1024));
      const uint32_t idesc_qk = p.idesc_qk, idesc_pv = p.idesc_pv;
      const uint64_t timeout_ns = p.timeout_ns;
      // A wait that fails (the CTA gave up somewhere) ends this role at once: nothing more is
      // issued on operands that never arrived.  All 32 lanes poll the same barrier, abort word and
      // timer in the same instructions, so the verdict is the same in every lane (the
      // elected-lane instructions below need the whole warp).
      bool ok = true;
      auto wait = [&](uint64_t* bar, uint32_t parity) -> bool {
        if (ok) ok = mbar_wait(bar, parity, abort_word, timeout_ns);
        return ok;
      };
      auto issue_qk = [&](uint32_t gi, int qb) {
        const int st = gi % ATTN_KV_STAGES;
        if (!wait(&k_full[st], (gi / ATTN_KV_STAGES) & 1u)) return;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (gi & 1u) * 128u;
        const uint32_t a0 = q_lo + static_cast<uint32_t>(qb) * TILE_UNITS;
        const uint32_t b0 = k_lo + static_cast<uint32_t>(st) * TILE_UNITS;
#pragma unroll
        for (int kk = 0; kk < ATTN_D / 16; ++kk) {
          // 16 elements along d are 32 bytes inside the 128-byte swizzle row; d 64..127 is the second box
          const uint32_t off = static_cast<uint32_t>((kk >> 2) * (TILE_UNITS / 2) + 2 * (kk & 3));
          if (elect_one()) umma_ss_words(d_tmem, a0 + off, desc_hi, b0 + off, desc_hi, idesc_qk, kk != 0 ? 1u : 0u);
        }
        if (elect_one()) {
          umma_commit(&k_empty[st]);
          umma_commit(&s_full[gi & 1u]);
        }
      };
      while (ok && cur.next(p, z, h, qt)) {
        if (*abort_word != 0) break;
        const AttnWave& w = p.waves[cur.wave];
        const int qpos0 = p.q_pos ? __ldg(p.q_pos + qt) : qt * ATTN_BM;
        int active = 0;
        for (int kb = w.kb0; kb < w.kb1; ++kb) active += block_mode(p, qpos0, kb) != 0;
        if (active == 0) continue;
        const int qb = u & 1;
        if (!wait(&q_full[qb], (u >> 1) & 1u)) break;
        issue_qk(g, qb);
        for (int j = 0; ok && j < active; ++j) {
          const uint32_t gi = g + j;
          if (j + 1 < active) issue_qk(gi + 1, qb);
          // P_j is in tensor memory (and O has been rescaled if the row maximum jumped)
          if (!wait(&p_full[gi & 1u], (gi >> 1) & 1u)) break;
          // the first product of a unit overwrites O: the previous unit's result must have been read
          if (j == 0 && !wait(&o_empty[0], (u & 1u) ^ 1u)) break;
          const int st = gi % ATTN_KV_STAGES;
          if (!wait(&v_full[st], (gi / ATTN_KV_STAGES) & 1u)) break;
          tc_fence_after();
          const uint32_t p_tmem = tmem_base + (gi & 1u) * 128u;  // bf16 pairs over the first 64 columns of S
          const uint32_t o_tmem = tmem_base + 256u;
          const uint32_t b0 = v_lo + static_cast<uint32_t>(st) * TILE_UNITS;
#pragma unroll
          for (int kk = 0; kk < ATTN_BN / 16; ++kk) {
            // V block in shared memory: [128 keys][64 d] per box, keys are the K axis (128 B apart),
            // d is the contiguous (MN) axis; the second box (d 64..127) lies 16 KB further
            if (elect_one())
              umma_ts_words(o_tmem, p_tmem + kk * 8, b0 + static_cast<uint32_t>(kk * 128), desc_hi, idesc_pv,
                            (j | kk) != 0 ? 1u : 0u);
          }
          if (elect_one()) {
            umma_commit(&v_empty[st]);
            umma_commit(&o_full[gi & 1u]);
          }
        }
        if (!ok) break;
        if (elect_one()) umma_commit(&q_empty[qb]);
        g += active;
        ++u;
      }
      if (__any_sync(0xffffffffu, *abort_word != 0)) {
        // products already issued still use shared and tensor memory: wait (bounded) until they
        // have completed before the CTA gives both back
        if (elect_one()) umma_commit(done_bar);
        drain_wait(done_bar, 0, timeout_ns);
      }
    }
  } else if (warp == 3) {
    if constexpr (FUSED) {
      comm_warp_run(p.comm, p.num_comm_ops, p.counters, p.signal_value, reinterpret_cast<char*>(ring), comm_bar,
                    abort_word, p.timeout_ns, lane);
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------ softmax / accumulate / merge / store
    const int q = warp & 3;
    const int row = q * 32 + lane;  // query row inside the tile, also the TMEM lane
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    UnitCursor cur;
    int z, h, qt;
    uint32_t g = 0;
    uint32_t u = 0;  // units processed (parity of the O hand-over barrier)
    // a wait that fails ends this role at once (the same verdict in every lane of a warp, which
    // polls in the same instructions; the tensor-memory instructions below are warp-wide);
    // nothing is stored for a unit that was not finished
    bool ok = true;
    auto wait = [&](uint64_t* bar, uint32_t parity) -> bool {
      if (ok) ok = mbar_wait(bar, parity, abort_word, p.timeout_ns);
      return ok;
    };
    while (ok && cur.next(p, z, h, qt)) {
      const AttnWave& w = p.waves[cur.wave];
      const int qpos0 = p.q_pos ? __ldg(p.q_pos + qt) : qt * ATTN_BM;
      int active = 0;
      for (int kb = w.kb0; kb < w.kb1; ++kb) active += block_mode(p, qpos0, kb) != 0;
      if (active == 0) continue;
      // m: maximum the stored P and O are scaled by; it follows the true row maximum lazily (only
      // when that has grown by more than 2^8), so that O in tensor memory is rarely rescaled
      float m = -INFINITY, l = 0.f;
      const uint32_t o_tmem = lane_base + 256u;
      int j = 0;
      for (int kb = w.kb0; kb < w.kb1; ++kb) {
        const int mode = block_mode(p, qpos0, kb);
        if (mode == 0) continue;
        const uint32_t gi = g + j;
        const uint32_t s_tmem = lane_base + (gi & 1u) * 128u;
        int lim = ATTN_BN - 1;  // keys 0..lim of the block are visible to this row
        if (mode == 2) {
          const int kpos0 = p.kv_pos ? __ldg(p.kv_pos + kb) : kb * ATTN_BN;
          lim = min(ATTN_BN - 1, qpos0 + row - kpos0);
        }
        if (!wait(&s_full[gi & 1u], (gi >> 1) & 1u)) break;
        tc_fence_after();
        // all of S for this row in one go: four loads in flight, one wait
        uint32_t sr[ATTN_BN / 32][32];
#pragma unroll
        for (int c = 0; c < ATTN_BN / 32; ++c) tmem_ld_32x32(s_tmem + c * 32, sr[c]);
        tmem_ld_wait();
        // eight independent chains: a single running maximum would serialise 128 dependent operations
        float mxs[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) mxs[i] = -INFINITY;
#pragma unroll
        for (int c = 0; c < ATTN_BN / 32; ++c) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (mode == 2 && c * 32 + i > lim) sr[c][i] = 0xff800000u;  // -inf
            mxs[i & 7] = fmaxf(mxs[i & 7], __uint_as_float(sr[c][i]));
          }
        }
        const float mx_raw = fmaxf(fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3])),
                                   fmaxf(fmaxf(mxs[4], mxs[5]), fmaxf(mxs[6], mxs[7])));
        const float mx = mx_raw * p.scale_log2;  // the scale is positive
        if (mx > m + 8.f) {
          // (first block, or the maximum jumped) move the reference point and rescale O and l
          if (j > 0 && m != -INFINITY) {
            // the previous product accumulates into O: it must be complete before O is touched.
            // (Nothing else needs this wait: by the time S of this block is full, every product
            // before the previous one has completed, and P of this block has a buffer of its own.)
            const uint32_t gp = gi - 1;
            mbar_wait(&o_full[gp & 1u], (gp >> 1) & 1u, abort_word, p.timeout_ns);
            tc_fence_after();
            const float alpha = exp2f(m - mx);
#pragma unroll 1
            for (int c = 0; c < ATTN_D / 32; ++c) {
              uint32_t r[32];
              tmem_ld_32x32(o_tmem + c * 32, r);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
              tmem_st_32x32(o_tmem + c * 32, r);
            }
            tmem_st_wait();
            l *= alpha;
          }
          m = mx;
        }
        const float neg_m = (m == -INFINITY) ? 0.f : -m;
        float ls[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < ATTN_BN / 32; ++c) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float p0 = ex2_approx(fmaf(__uint_as_float(sr[c][2 * i]), p.scale_log2, neg_m));
            const float p1 = ex2_approx(fmaf(__uint_as_float(sr[c][2 * i + 1]), p.scale_log2, neg_m));
            ls[i & 3] += p0 + p1;
            pk[i] = BF16 ? pack2_bf16(p0, p1) : pack2_f16(p0, p1);
          }
          tmem_st_32x16(s_tmem + c * 16, pk);
        }
        l += (ls[0] + ls[1]) + (ls[2] + ls[3]);
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(&p_full[gi & 1u]);
        ++j;
      }
      if (!ok) break;
      // the unit's last product
      {
        const uint32_t gp = g + active - 1;
        if (!wait(&o_full[gp & 1u], (gp >> 1) & 1u)) break;
        tc_fence_after();
      }
      g += active;

      attn_finish_row<BF16>(p, z, h, qt, row, m, l, o_tmem);
      // O has been read: the next unit's first product may overwrite it
      tc_fence_before();
      mbar_arrive(&o_empty[0]);
      ++u;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_word != 0 && p.status != nullptr) {
    if (atomicCAS(p.status, 0, *abort_word) == 0) {
      p.status[1] = abort_info[0];
      p.status[2] = abort_info[1];
      p.status[3] = static_cast<int>(blockIdx.x);
    }
  }
}

}  // namespace syn
