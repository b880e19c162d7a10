// Two-tile form of the flash-attention forward kernel: a CTA works on two adjacent 128-row query
// tiles (A = 2u, B = 2u + 1) at a time.  They share every K / V block brought into shared memory,
// and each has a softmax warpgroup of its own, so two warps per scheduler overlap each other's
// exponentials, conversions and tensor-memory traffic, and the tensor pipe runs one tile's
// products while the other tile is in its softmax.
//
// Same semantics as attn_kernel (waves in order, flags, causal masking by true positions, grouped
// heads, log-sum-exp merge over waves by fixed ownership); the ownership unit is the tile pair.
//
// Tensor memory (512 columns): S_A 0..127, S_B 128..255, O_A 256..383, O_B 384..511; P overwrites
// the first 64 columns of its S.  A tile has ONE S buffer: its next S = Q K^T is issued right after
// its P V, and the other tile's work fills the tensor pipe meanwhile.  Each tile has an issuing
// warp of its own; per key block j it runs
//   wait P_X(j) [first half]; O_X += P_X(j) V(j) [keys 0..63]; wait P_X(j) [second half];
//   O_X += P_X(j) V(j) [keys 64..127]; S_X = Q_X K(j+1)^T
// The commit that publishes S_X(j+1) follows P_X(j) V(j) in issue order, so a softmax thread that
// sees S full knows the previous product into O_X has completed and may rescale O_X at once.
//
// Roles (384 threads): warp 0 TMA producer, warps 1 and 2 MMA issuers of tile A and tile B (warp 2
// also allocates the tensor memory), warp 3 comm warp (optional), warps 4-7 softmax of tile A,
// warps 8-11 softmax of tile B.  The first warpgroup
// gives registers up (setmaxnreg) so that a softmax thread can hold a whole row of S.
#pragma once
#include "attn_sm100.cuh"

namespace syn {

constexpr int ATTN2_THREADS = 384;
// Register split between the first warpgroup (producer, MMA issuer, allocator, comm warp) and the
// two softmax warpgroups.  setmaxnreg only moves registers inside what the CTA was launched with
// (168 per thread under __launch_bounds__(384, 1)); asking for more makes the increase wait for
// ever, so the sum is checked here.
#define SYN_ATTN2_REGS_LOW 88
#define SYN_ATTN2_REGS_HIGH 208
static_assert(128 * SYN_ATTN2_REGS_LOW + 256 * SYN_ATTN2_REGS_HIGH <= 168 * ATTN2_THREADS,
              "setmaxnreg split exceeds the registers the CTA owns");
#define SYN_STR2(x) #x
#define SYN_STR(x) SYN_STR2(x)

// What one tile of the pair does in one wave.
struct TileRole {
  bool in_wave;
  int qt;      // query tile index
  int qpos0;   // true position of its first row
};
__device__ __forceinline__ TileRole tile_role(const AttnParams& p, const AttnWave& w, int qt) {
  TileRole t;
  t.qt = qt;
  t.in_wave = qt >= w.q0t && qt < w.q0t + w.nqt;
  t.qpos0 = !t.in_wave ? 0 : (p.q_pos ? __ldg(p.q_pos + qt) : qt * ATTN_BM);
  return t;
}
__device__ __forceinline__ int tile_mode(const AttnParams& p, const TileRole& t, int kb) {
  return t.in_wave ? block_mode(p, t.qpos0, kb) : 0;
}
// First key block at or after `from` that either tile needs (-1 = none), with both tiles' modes.
__device__ __forceinline__ int next_shared_block(const AttnParams& p, const AttnWave& w, const TileRole& a,
                                                 const TileRole& b, int from, int& ma, int& mb) {
  for (int kb = from; kb < w.kb1; ++kb) {
    ma = tile_mode(p, a, kb);
    mb = tile_mode(p, b, kb);
    if ((ma | mb) != 0) return kb;
  }
  ma = mb = 0;
  return -1;
}

// Packed pairs of fp32 (one 64-bit register) for the two-wide fp32 instructions of sm_100.
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

template <bool FUSED, bool BF16>
__global__ void __launch_bounds__(ATTN2_THREADS, 1) attn2_kernel(const __grid_constant__ AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                                        // tile A, tile B
  uint8_t* sK = sQ + 2 * ATTN_TILE_BYTES;                    // ATTN_KV_STAGES blocks
  uint8_t* sV = sK + ATTN_KV_STAGES * ATTN_TILE_BYTES;       // ATTN_KV_STAGES blocks
  uint8_t* ring = sV + ATTN_KV_STAGES * ATTN_TILE_BYTES;     // FUSED only
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring + (FUSED ? COMM_NBUF * COMM_PIECE : 0));
  uint64_t* q_full = bars;            // [2] per tile
  uint64_t* q_empty = bars + 2;       // [2]
  uint64_t* k_full = bars + 4;        // [KV_STAGES]
  uint64_t* k_empty = bars + 6;
  uint64_t* v_full = bars + 8;
  uint64_t* v_empty = bars + 10;
  uint64_t* s_full = bars + 12;       // [2] per tile, MMA -> softmax
  uint64_t* p_full = bars + 14;       // [2][2] per tile and half of P (keys 0..63 / 64..127), softmax -> MMA
  uint64_t* o_full = bars + 18;       // [2] per tile, MMA -> softmax, once per unit
  uint64_t* o_empty = bars + 20;      // [2] per tile, softmax -> MMA, once per unit
  uint64_t* turn = bars + 22;         // [2] per tile: its softmax warpgroup may exponentiate
  uint64_t* comm_bar = bars + 24;     // [COMM_NBUF]
  uint64_t* done_bar = bars + 24 + COMM_NBUF;  // [2] per issuing warp: its products have completed (give-up path)
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 26 + COMM_NBUF);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_holder + 1);
  int* abort_info = const_cast<int*>(abort_word) + 1;
  // producer role: visits left per (unit of this CTA's list, tile)
  volatile uint8_t* left = reinterpret_cast<volatile uint8_t*>(abort_info + 2);
  const bool pushing = p.num_push > 0;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (pushing && threadIdx.x >= 128 && threadIdx.x < 128 + 2 * ATTN_PUSH_MAX_UNITS_PER_CTA) {
    const int idx = threadIdx.x - 128, first = p.own_start[blockIdx.x], count = p.own_start[blockIdx.x + 1] - first;
    left[idx] = (idx >> 1) < count ? p.visits[2 * p.own_units[first + (idx >> 1)] + (idx & 1)] : 0;
  }
  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      // with the producer role the softmax warpgroup stages its last rows in the Q tile's shared
      // memory, so it (and not the issuer's last product) hands the tile back to the loader
      mbar_init(&q_empty[i], pushing ? 128 : 1);
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 2);  // one release per MMA warp
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 2);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[2 * i], 128);
      mbar_init(&p_full[2 * i + 1], 128);
      mbar_init(&o_full[i], 1);
      mbar_init(&o_empty[i], 128);
      mbar_init(&turn[i], 128);
    }
    for (int i = 0; i < COMM_NBUF; ++i) mbar_init(&comm_bar[i], 1);
    mbar_init(&done_bar[0], 1);
    mbar_init(&done_bar[1], 1);
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

  if (warp < 4) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 " SYN_STR(SYN_ATTN2_REGS_LOW) ";");
  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      UnitCursor cur;
      cur.shift = 1;
      int z, h, un;
      uint32_t uq[2] = {0, 0};  // units each tile has taken part in (parity of its Q barriers)
      uint32_t g = 0;           // shared key blocks loaded so far (ring position)
      int flag_wave = -1;
      uint32_t kfills = 0, vfills = 0;  // K / V loads issued (a give-up may fall between the two)
      bool ok = true;
      while (ok && cur.next(p, z, h, un)) {
        if (*abort_word != 0) break;
        const AttnWave& w = p.waves[cur.wave];
        const TileRole ta = tile_role(p, w, 2 * un), tb = tile_role(p, w, 2 * un + 1);
        int act[2] = {0, 0};
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          act[0] += tile_mode(p, ta, kb) != 0;
          act[1] += tile_mode(p, tb, kb) != 0;
        }
        if (act[0] + act[1] == 0) continue;
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
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          if (act[x] == 0 || !ok) continue;
          const int qt = 2 * un + x;
          if (!mbar_wait(&q_empty[x], (uq[x] & 1u) ^ 1u, abort_word, p.timeout_ns)) {
            ok = false;
            continue;
          }
          mbar_expect_tx(&q_full[x], ATTN_TILE_BYTES);
          tma_load_4d(sQ + x * ATTN_TILE_BYTES, &p.tmap_q, &q_full[x], 0, qt * ATTN_BM, h, z);
          tma_load_4d(sQ + x * ATTN_TILE_BYTES + ATTN_TILE_BYTES / 2, &p.tmap_q, &q_full[x], 64, qt * ATTN_BM, h, z);
          ++uq[x];
        }
        const int hk = h / group;
        int ma, mb;
        for (int kb = next_shared_block(p, w, ta, tb, w.kb0, ma, mb); ok && kb >= 0;
             kb = next_shared_block(p, w, ta, tb, kb + 1, ma, mb)) {
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
        for (int x = 0; x < 2; ++x) drain_stage(&q_full[x], uq[x], p.timeout_ns);
        for (int st = 0; st < ATTN_KV_STAGES; ++st) {
          drain_stage(&k_full[st], kfills / ATTN_KV_STAGES + (static_cast<uint32_t>(st) < kfills % ATTN_KV_STAGES ? 1u : 0u),
                      p.timeout_ns);
          drain_stage(&v_full[st], vfills / ATTN_KV_STAGES + (static_cast<uint32_t>(st) < vfills % ATTN_KV_STAGES ? 1u : 0u),
                      p.timeout_ns);
        }
      }
    }
  } else if (warp == 1 || warp == 2) {
    // ------------------------------------------------------------ MMA issuers: warp 1 for tile A, warp 2 for tile B
    // A warp walks the schedule and waits on the barriers as a whole; one elected lane issues each
    // tcgen05 instruction.  (A single diverged lane that also computes the descriptors is several
    // times slower per instruction, and one warp serving both tiles spends more time in its waits
    // than the tensor pipe needs for the work.)  Both warps see every shared key block: the one
    // whose tile skips a block releases its K / V stage with a plain arrive.
    {
      const int x = warp - 1;
      UnitCursor cur;
      cur.shift = 1;
      int z, h, un;
      uint32_t uqx = 0;  // units of this tile (Q and O barriers)
      uint32_t cbx = 0;  // key blocks of this tile (S and P barriers)
      uint32_t g = 0;    // shared key blocks (K / V ring)
      const uint64_t timeout_ns = p.timeout_ns;
      // descriptor words: the low word carries the address in 16-byte units (and the leading
      // offset), the high word the stride between 8-row groups, the version and the swizzle mode
      constexpr uint32_t TILE_UNITS = ATTN_TILE_BYTES >> 4;
      const uint32_t desc_hi = static_cast<uint32_t>(make_smem_desc_sw128(0, 16, 1024) >> 32);
      const uint32_t q_lo = static_cast<uint32_t>(make_smem_desc_sw128(smem_u32(sQ), 16, 1024)) +
                            static_cast<uint32_t>(x) * TILE_UNITS;
      const uint32_t k_lo = static_cast<uint32_t>(make_smem_desc_sw128(smem_u32(sK), 16, 1024));
      const uint32_t v_lo = static_cast<uint32_t>(make_smem_desc_sw128(smem_u32(sV), ATTN_TILE_BYTES / 2, 1024));
      const uint32_t s_tmem = tmem_base + static_cast<uint32_t>(x) * 128u;  // S_x, then P_x
      const uint32_t o_tmem = tmem_base + 256u + static_cast<uint32_t>(x) * 128u;
      const uint32_t idesc_qk = p.idesc_qk, idesc_pv = p.idesc_pv;
      // A wait that fails (the CTA gave up somewhere) ends this role at once: nothing more is
      // issued on operands that never arrived.  All 32 lanes poll the same barrier, abort word and
      // timer in the same instructions, so the verdict is the same in every lane (the
      // elected-lane instructions below need the whole warp).
      bool ok = true;
      auto wait = [&](uint64_t* bar, uint32_t parity) -> bool {
        if (ok) ok = mbar_wait(bar, parity, abort_word, timeout_ns);
        return ok;
      };
      // S_x = Q_x K^T for the block in K stage `st`
      auto issue_qk = [&](int st) {
        const uint32_t b0 = k_lo + static_cast<uint32_t>(st) * TILE_UNITS;
        // (electing once around the whole group was measured slower: the descriptor words then
        // live in per-lane registers of a diverged lane)
#pragma unroll
        for (int kk = 0; kk < ATTN_D / 16; ++kk) {
          // 16 elements along d are 32 bytes inside the 128-byte swizzle row; d 64..127 is the second box
          const uint32_t off = static_cast<uint32_t>((kk >> 2) * (TILE_UNITS / 2) + 2 * (kk & 3));
          if (elect_one()) umma_ss_words(s_tmem, q_lo + off, desc_hi, b0 + off, desc_hi, idesc_qk, kk != 0 ? 1u : 0u);
        }
        if (elect_one()) umma_commit(&s_full[x]);
      };
      // O_x (+)= P_x V for one half (64 keys) of the block in V stage `st`
      auto issue_pv = [&](int st, int half, bool accumulate) {
        const uint32_t b0 = v_lo + static_cast<uint32_t>(st) * TILE_UNITS;
#pragma unroll
        for (int k4 = 0; k4 < ATTN_BN / 32; ++k4) {
          const int kk = half * (ATTN_BN / 32) + k4;
          // V block: [128 keys][64 d] per box, keys are the K axis (128 B apart), d is the contiguous
          // (MN) axis; the second box (d 64..127) lies 16 KB further (the leading offset)
          if (elect_one())
            umma_ts_words(o_tmem, s_tmem + kk * 8, b0 + static_cast<uint32_t>(kk * 128), desc_hi, idesc_pv,
                          (accumulate || kk != 0) ? 1u : 0u);
        }
      };
      // stage release: after this warp's products if it issued any, at once otherwise
      auto release = [&](uint64_t* bar, bool issued) {
        if (elect_one()) {
          if (issued) {
            umma_commit(bar);
          } else {
            mbar_arrive(bar);
          }
        }
      };
      while (ok && cur.next(p, z, h, un)) {
        if (*abort_word != 0) break;
        const AttnWave& w = p.waves[cur.wave];
        const TileRole tr[2] = {tile_role(p, w, 2 * un), tile_role(p, w, 2 * un + 1)};
        int act[2] = {0, 0};
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          act[0] += tile_mode(p, tr[0], kb) != 0;
          act[1] += tile_mode(p, tr[1], kb) != 0;
        }
        if (act[0] + act[1] == 0) continue;
        if (act[x] && !wait(&q_full[x], uqx & 1u)) break;
        int m[2], n[2];
        int kb = next_shared_block(p, w, tr[0], tr[1], w.kb0, m[0], m[1]);
        // the unit's first block
        {
          const int st = g % ATTN_KV_STAGES;
          // (a warp whose tile skips the block still waits for the stage to be full before it
          // releases it: otherwise it could run ahead and arrive twice in one phase)
          if (!wait(&k_full[st], (g / ATTN_KV_STAGES) & 1u)) break;
          if (m[x]) {
            tc_fence_after();
            issue_qk(st);
          }
          release(&k_empty[st], m[x] != 0);
        }
        bool started = false;
        while (ok && kb >= 0) {
          const int kn = next_shared_block(p, w, tr[0], tr[1], kb + 1, n[0], n[1]);
          const int st = g % ATTN_KV_STAGES, st_n = (g + 1) % ATTN_KV_STAGES;
          const uint32_t par = (g / ATTN_KV_STAGES) & 1u, par_n = ((g + 1) / ATTN_KV_STAGES) & 1u;
          if (m[x]) {
            if (!wait(&p_full[2 * x], cbx & 1u)) break;
            // the first product of a unit overwrites O_x: the previous unit's result must have been read
            if (!started && !wait(&o_empty[x], (uqx & 1u) ^ 1u)) break;
            if (!wait(&v_full[st], par)) break;
            tc_fence_after();
            issue_pv(st, 0, started);
            // the next K block has long landed; looking now keeps this wait off the path from the
            // second half of P to the next S
            if (kn >= 0 && !wait(&k_full[st_n], par_n)) break;
            if (!wait(&p_full[2 * x + 1], cbx & 1u)) break;
            tc_fence_after();
            issue_pv(st, 1, true);
            ++cbx;
            started = true;
            if (kn >= 0 && n[x]) {
              issue_qk(st_n);
            }
            // both stages are released by one commit each, after everything issued so far
            release(&v_empty[st], true);
            if (kn >= 0) release(&k_empty[st_n], n[x] != 0);
          } else {
            if (!wait(&v_full[st], par)) break;
            release(&v_empty[st], false);
            if (kn >= 0) {
              if (!wait(&k_full[st_n], par_n)) break;
              if (n[x]) {
                tc_fence_after();
                issue_qk(st_n);
              }
              release(&k_empty[st_n], n[x] != 0);
            }
          }
          kb = kn;
          m[0] = n[0];
          m[1] = n[1];
          ++g;
        }
        if (!ok) break;
        if (act[x]) {
          if (elect_one()) {
            umma_commit(&o_full[x]);
            if (!pushing) umma_commit(&q_empty[x]);
          }
          ++uqx;
        }
      }
      if (__any_sync(0xffffffffu, *abort_word != 0)) {
        // products already issued still use shared and tensor memory: wait (bounded) until they
        // have completed before the CTA gives both back
        if (elect_one()) umma_commit(&done_bar[x]);
        drain_wait(&done_bar[x], 0, timeout_ns);
      }
    }
  } else if (warp == 3) {
    if constexpr (FUSED) {
      comm_warp_run(p.comm, p.num_comm_ops, p.counters, p.signal_value, reinterpret_cast<char*>(ring), comm_bar,
                    abort_word, p.timeout_ns, lane);
    }
  }
  } else {
    // ------------------------------------------------------------ softmax / accumulate / merge / store
    asm volatile("setmaxnreg.inc.sync.aligned.u32 " SYN_STR(SYN_ATTN2_REGS_HIGH) ";");
    const int x = (warp >= 8) ? 1 : 0;  // which tile of the pair
    const int q = warp & 3;
    const int row = q * 32 + lane;      // query row inside the tile, also the TMEM lane
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    const uint32_t s_tmem = lane_base + static_cast<uint32_t>(x) * 128u;
    const uint32_t o_tmem = lane_base + 256u + static_cast<uint32_t>(x) * 128u;
    UnitCursor cur;
    cur.shift = 1;
    int z, h, un;
    uint32_t cbx = 0;  // key blocks this tile has processed (S / P barrier parity)
    uint32_t ux = 0;   // units this tile has taken part in
    uint32_t turns = 0;  // blocks both tiles have worked on (parity of the turn barriers)
    // a wait that fails ends this role at once (the same verdict in every lane of a warp, which
    // polls in the same instructions; the tensor-memory instructions below are warp-wide);
    // nothing is stored for a unit that was not finished
    bool ok = true;
    auto wait = [&](uint64_t* bar, uint32_t parity) -> bool {
      if (ok) ok = mbar_wait(bar, parity, abort_word, p.timeout_ns);
      return ok;
    };
    while (ok && cur.next(p, z, h, un)) {
      // (with the producer role the four warps of a tile leave together, at the unit's closing barrier)
      if (!pushing && *abort_word != 0) break;
      const AttnWave& w = p.waves[cur.wave];
      const TileRole t = tile_role(p, w, 2 * un + x), other = tile_role(p, w, 2 * un + (x ^ 1));
      int active = 0;
      for (int kb = w.kb0; kb < w.kb1; ++kb) active += tile_mode(p, t, kb) != 0;
      if (active == 0) continue;
      const int qt = t.qt, qpos0 = t.qpos0;
      // m: maximum the stored P and O are scaled by; it follows the true row maximum lazily (only
      // when that has grown by more than 2^8), so that O in tensor memory is rarely rescaled
      float m = -INFINITY, l = 0.f;
      int j = 0;
      for (int kb = w.kb0; kb < w.kb1; ++kb) {
        const int mode = block_mode(p, qpos0, kb);
        if (mode == 0) continue;
        const bool both = tile_mode(p, other, kb) != 0;  // the other tile works on this block too
        int lim = ATTN_BN - 1;  // keys 0..lim of the block are visible to this row
        if (mode == 2) {
          const int kpos0 = p.kv_pos ? __ldg(p.kv_pos + kb) : kb * ATTN_BN;
          lim = min(ATTN_BN - 1, qpos0 + row - kpos0);
        }
        if (!wait(&s_full[x], cbx & 1u)) break;
        ++cbx;
        tc_fence_after();
        uint32_t sr[ATTN_BN / 32][32];
#pragma unroll
        for (int c = 0; c < ATTN_BN / 32; ++c) tmem_ld_32x32(s_tmem + c * 32, sr[c]);
        tmem_ld_wait();
        if (mode == 2) {
#pragma unroll
          for (int c = 0; c < ATTN_BN / 32; ++c) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (c * 32 + i > lim) sr[c][i] = 0xff800000u;  // -inf
          }
        }
        // four independent chains of three-input maxima
        float mxs[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int c = 0; c < ATTN_BN / 32; ++c) {
#pragma unroll
          for (int i = 0; i < 16; ++i)
            mxs[i & 3] = fmax3(mxs[i & 3], __uint_as_float(sr[c][2 * i]), __uint_as_float(sr[c][2 * i + 1]));
        }
        const float mx_raw = fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3]));
        const float mx = mx_raw * p.scale_log2;  // the scale is positive
        if (mx > m + 8.f) {
          // (first block, or the maximum jumped) move the reference point and rescale O and l; the
          // previous product into O has completed (its commit precedes the one that published S)
          if (j > 0 && m != -INFINITY) {
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
            l *= alpha;
          }
          m = mx;
        }
        const float neg_m = (m == -INFINITY) ? 0.f : -m;
        // P = 2^(S * scale - m), two elements per instruction where the hardware allows; the two
        // halves of P (keys 0..63, 64..127) are handed over separately, so that the product with
        // the first half of V runs while the second half is still being exponentiated
        // The two warpgroups take turns at the exponentials (A, B, A, B ... over the blocks both
        // work on): the special-function unit serves one of them at full rate instead of both at
        // half, and the tiles settle half a period apart, so that one tile's products run on the
        // tensor pipe during the other tile's softmax.
        if (both && !wait(&turn[x], x == 0 ? ((turns & 1u) ^ 1u) : (turns & 1u))) break;
        const uint64_t scale2 = f2_pack(p.scale_log2, p.scale_log2), negm2 = f2_pack(neg_m, neg_m);
        uint64_t ls2[2] = {0ull, 0ull};  // packed (0.f, 0.f)
        // One chunk = 32 values: scale (packed FMA) and exponentiate in place.  The exponentials of
        // chunk c + 1 are issued BEFORE chunk c is summed, packed and stored, so that those consumers
        // sit in the same instruction window as the next chunk's independent exponentials (measured
        // neutral at S = 32768: 1.0147 ms with, 1.0146 ms without).
        auto scale_exp = [&](int c) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            float x0, x1;
            f2_unpack(f2_fma(f2_pack(__uint_as_float(sr[c][2 * i]), __uint_as_float(sr[c][2 * i + 1])), scale2, negm2),
                      x0, x1);
            sr[c][2 * i] = __float_as_uint(x0);
            sr[c][2 * i + 1] = __float_as_uint(x1);
          }
#pragma unroll
          for (int i = 0; i < 32; ++i) sr[c][i] = __float_as_uint(ex2_approx(__uint_as_float(sr[c][i])));
        };
        scale_exp(0);
#pragma unroll
        for (int c = 0; c < ATTN_BN / 32; ++c) {
          if (c + 1 < ATTN_BN / 32) scale_exp(c + 1);
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float p0 = __uint_as_float(sr[c][2 * i]), p1 = __uint_as_float(sr[c][2 * i + 1]);
            ls2[i & 1] = f2_add(ls2[i & 1], f2_pack(p0, p1));
            pk[i] = BF16 ? pack2_bf16(p0, p1) : pack2_f16(p0, p1);
          }
          tmem_st_32x16(s_tmem + c * 16, pk);
          if (c & 1) {
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(&p_full[2 * x + (c >> 1)]);
          }
        }
        if (both) {
          mbar_arrive(&turn[x ^ 1]);
          ++turns;
        }
        {
          float a0, a1, b0, b1;
          f2_unpack(ls2[0], a0, a1);
          f2_unpack(ls2[1], b0, b1);
          l += (a0 + a1) + (b0 + b1);
        }
        ++j;
      }
      if (!pushing) {
        if (!ok) break;
        // the unit's last product into O_x
        if (!wait(&o_full[x], ux & 1u)) break;
        tc_fence_after();

        attn_finish_row<BF16>(p, z, h, qt, row, m, l, o_tmem);
        // O_x has been read: the next unit's first product may overwrite it
        tc_fence_before();
        mbar_arrive(&o_empty[x]);
        ++ux;
        continue;
      }
      // ---- producer role.  The tile's four warps meet at a barrier that also tells them whether
      // any of them gave up, so that they leave the loop at the same unit.
      const int pos = cur.slot - 1 - static_cast<int>(p.own_start[blockIdx.x]);
      const bool last_visit = left[2 * pos + x] == 1;
      int slab = 0;
      if (ok) wait(&o_full[x], ux & 1u);
      if (ok) {
        tc_fence_after();
        // The tile's last visit: its final rows (merged with what earlier visits left in `o`) are
        // staged in the Q tile's shared memory, which nothing reads any more, and leave as two TMA
        // stores per warp into the destination rank's buffer.
        uint8_t* stage = last_visit ? sQ + x * ATTN_TILE_BYTES + q * 8192 : nullptr;
        attn_finish_row<BF16>(p, z, h, qt, row, m, l, o_tmem, stage);
        if (last_visit) {
          while (slab + 1 < p.num_push && qt * ATTN_BM >= p.push[slab].s1) ++slab;
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            const int drow = p.push[slab].row0 + (qt * ATTN_BM - p.push[slab].s0) + q * 32;
            tma_store_4d(&p.tmap_push[slab], stage, 0, drow, p.push_head0 + h, z);
            tma_store_4d(&p.tmap_push[slab], stage + 4096, 64, drow, p.push_head0 + h, z);
            bulk_commit();
            bulk_wait<0>();       // landed (not just read): the slab's flag may follow
            fence_proxy_async();
            __threadfence_system();
          }
        }
        tc_fence_before();
      }
      uint32_t anybody_failed;
      asm volatile(
          "{\n"
          ".reg .pred pin, pout;\n"
          "setp.ne.u32 pin, %1, 0;\n"
          "barrier.cta.red.or.pred pout, %2, 128, pin;\n"
          "selp.u32 %0, 1, 0, pout;\n"
          "}\n"
          : "=r"(anybody_failed)
          : "r"(ok ? 0u : 1u), "r"(2 + x)
          : "memory");
      if (anybody_failed) {
        ok = false;
        break;
      }
      if ((threadIdx.x & 127) == 0) {
        left[2 * pos + x] = static_cast<uint8_t>(left[2 * pos + x] - 1);
        if (last_visit) {
          // every warp's stores have landed (they waited before the barrier): count the tile in
          const AttnPushSlab& ps = p.push[slab];
          __threadfence_system();
          const uint32_t old = atomicAdd(&p.push_counters[slab], 1u);
          if (old + 1u == static_cast<uint32_t>(ps.tiles)) {
            p.push_counters[slab] = 0;
            __threadfence_system();
            if (ps.flag != nullptr) st_release_sys_u64(ps.flag, p.signal_value);
          }
        }
      }
      mbar_arrive(&q_empty[x]);  // the staging space is the loader's again
      mbar_arrive(&o_empty[x]);  // O_x has been read: the next unit's first product may overwrite it
      ++ux;
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
