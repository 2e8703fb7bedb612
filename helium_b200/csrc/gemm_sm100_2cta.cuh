// Two-CTA variant of the tcgen05 GEMM core: a cluster of two CTAs (two SMs) works on one
// 256 x 256 output tile with `tcgen05.mma.cta_group::2`.  Each CTA owns 128 rows of A (and of the
// mainloop mask) and loads only half of the B tile (128 of the 256 columns); the tensor cores of
// both SMs read both halves.  Per SM and k-block that is 32 KB of operands instead of 48 KB
// (48 KB instead of 64 KB with a mask tile), which is what the L2 -> SM path can sustain, and the
// shared-memory ring gets six stages instead of four (four instead of three with a mask).
//
// Every load is a per-CTA TMA load: each CTA fetches its own boxes with `.cta_group::2` loads
// whose mbarrier is the leader CTA's.  Cross-CTA signalling uses remote mbarrier arrives and
// `tcgen05.commit` to the peer's barrier.
#pragma once
#include "gemm_sm100.cuh"

namespace he {
namespace ptx {

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t mapa(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
// Arrive on an mbarrier of a CTA of this cluster (address from mapa).  Default semantics on purpose:
// spelling out `.release.cluster` made every transform-warp hand-off of the fused mainloop about
// 1 us slower (678 -> 383 TFLOP/s on the mainloop-fused 4096^3 case); the shared-memory writes that
// the arrival publishes are ordered for the tensor core by the async-proxy fence issued before it.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_load_3d_2cta(uint32_t dst, const CUtensorMap* m, uint32_t leader_bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(leader_bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_2cta(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_2cta() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc_2cta(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f16_2cta(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_f8_2cta(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
      "}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// `bar` is a shared::cluster address (own or peer CTA)
__device__ __forceinline__ void umma_commit_2cta(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

}  // namespace ptx

constexpr int kBN2 = 256;            // N of the pair tile
constexpr int kBHalfBytes = 128 * kBK * 2;   // this CTA's half of the B tile: 16 KiB

template <int STAGES, int ML, int N_COLRED>
struct GemmSmem2 {
  static constexpr bool kHasMask = (ML & ML_MASK) != 0;
  static constexpr int off_a = 0;
  static constexpr int off_b = off_a + STAGES * kATileBytes;
  static constexpr int off_mask = off_b + STAGES * kBHalfBytes;
  static constexpr int off_scratch = off_mask + (kHasMask ? STAGES * kATileBytes : 0);
  static constexpr int scratch_bytes = (N_COLRED * 4 * kBN2 + 64) * 4;
  static constexpr int off_bar = off_scratch + scratch_bytes;
  // full_b[S] (leader), full_a[S] (local, mainloop fusion only), empty[S] (local), xform[S] (leader),
  // tmem_full[2] (local), tmem_empty[2] (leader)
  static constexpr int n_bars = 4 * STAGES + 4;
  static constexpr int off_misc = off_bar + n_bars * 8;
  static constexpr int total = off_misc + 16;
  static constexpr int dynamic_bytes = total + 1024;
};

template <int STAGES, bool A_MN, bool B_MN, int ML, int NE_WARPS, class Epi>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(32 * (2 + NE_WARPS + (ml_transforms(ML) ? 4 : 0)), 1)
gemm_tcgen05_2cta_kernel(const __grid_constant__ GemmParams<typename Epi::Params> p) {
  using SM = GemmSmem2<STAGES, ML, Epi::kColReductions>;
  constexpr int BN = kBN2;
  constexpr int kXformWarp0 = 2 + NE_WARPS;
  constexpr int kTmemCols = 512;
  constexpr int CH = Epi::kChunk;
  constexpr bool kFused = ml_transforms(ML);
  // Plain mainloops hand shared memory over in units of TWO k-blocks (64 KB per CTA): one barrier wait, one
  // expect_tx and one pair of commits per eight MMAs instead of per four.  The MMA-issuing thread spends ~65 cycles
  // per MMA and ~280 per hand-over; with four MMAs (512 tensor-pipe cycles) per hand-over it, not the tensor pipe,
  // set the pace.  The rewriting mainloops keep one k-block per hand-over (their transform warps pace them).
  constexpr int KSUB = kFused ? 1 : 2;
  constexpr int GROUPS = STAGES / KSUB;
  static_assert(STAGES % KSUB == 0, "stages are handed over in groups of KSUB");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t smem_base = ptx::smem_u32(smem);
  const uint32_t bar0 = smem_base + SM::off_bar;
  auto bar_full_b = [&](int s) { return bar0 + 8u * s; };
  auto bar_full_a = [&](int s) { return bar0 + 8u * (STAGES + s); };
  auto bar_empty = [&](int s) { return bar0 + 8u * (2 * STAGES + s); };
  auto bar_xform = [&](int s) { return bar0 + 8u * (3 * STAGES + s); };
  auto bar_tmem_full = [&](int a) { return bar0 + 8u * (4 * STAGES + a); };
  auto bar_tmem_empty = [&](int a) { return bar0 + 8u * (4 * STAGES + 2 + a); };
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(smem + SM::off_misc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM::off_misc + 4);
  float* scratch = reinterpret_cast<float*>(smem + SM::off_scratch);

  const GemmCore& c = p.core;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();   // 0 = leader
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int tiles_m2 = (c.M + 255) / 256;
  // The tile list: every 256 x 256 pair tile once, except that the last `split_count` of them
  // appear as two 256 x 128 halves.  With 256 tiles on 74 pairs the fourth round would keep 34 pairs
  // busy and 40 idle; as 68 half tiles it keeps 68 busy for about half as long.
  const int pair_tiles = tiles_m2 * c.tiles_n * c.batch + c.split_count;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(bar_full_b(s), 1);          // leader's arrive.expect_tx; bytes from both CTAs
      ptx::mbar_init(bar_full_a(s), 1);          // local arrive.expect_tx (A + mask of this CTA)
      ptx::mbar_init(bar_empty(s), 1);           // one tcgen05.commit per CTA, issued by the leader
      ptx::mbar_init(bar_xform(s), 2 * 4);       // one arrival per transform warp of both CTAs
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(bar_tmem_full(a), 1);
      ptx::mbar_init(bar_tmem_empty(a), 2 * NE_WARPS);   // one arrival per epilogue warp of both CTAs
    }
    ptx::fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    ptx::prefetch_tmap(&p.tma_a);
    ptx::prefetch_tmap(&p.tma_b);
    if (SM::kHasMask) ptx::prefetch_tmap(&p.tma_mask);
  }
  if (warp == 1) {
    ptx::tmem_alloc_2cta(ptx::smem_u32(const_cast<uint32_t*>(tmem_holder)), kTmemCols);
    ptx::tmem_relinquish_2cta();
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::cluster_sync();   // both CTAs' barriers are initialised before anyone signals across
  ptx::tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  // pair tile -> (batch, m2, n); this CTA's rows start at m2 * 256 + rank * 128
  auto decode_tile = [&](int list_idx) {
    TileInfo t;
    int tile = list_idx, half = -1;
    if (list_idx >= c.split_from && c.split_count > 0) {
      const int h = list_idx - c.split_from;
      tile = c.split_from + (h >> 1);
      half = h & 1;
    }
    const int per_batch = tiles_m2 * c.tiles_n;
    t.b = tile / per_batch;
    const int r = tile - t.b * per_batch;
    const int gsz = c.group_m * c.tiles_n;   // group_m counts 256-row pair tiles here
    const int g = r / gsz;
    const int first_m = g * c.group_m;
    const int gm = min(c.group_m, tiles_m2 - first_m);
    const int w = r - g * gsz;
    t.tile_n = w / gm;
    const int m2 = first_m + (w - t.tile_n * gm);
    t.tile_m = m2 * 2 + (int)rank;
    t.m0 = t.tile_m * kBM;
    t.n0 = t.tile_n * BN + (half > 0 ? BN / 2 : 0);
    t.bn = half >= 0 ? BN / 2 : BN;
    t.tile_idx = list_idx * 2 + (int)rank;
    return t;
  };

  if (warp == 0) {
    // ===================== TMA producer (both CTAs) =====================
    if (lane == 0) {
      constexpr uint32_t kABytes = kATileBytes + (SM::kHasMask ? kATileBytes : 0);
      // bytes the leader's barrier sees per stage: both B halves, plus both A tiles when they are
      // not routed through the local barrier
      constexpr uint32_t kLeaderBytes = 2 * kBHalfBytes + (kFused ? 0 : 2 * kATileBytes);
      int stage = 0;
      uint32_t phase = 0;
      bool alive = true;
      int it = 0;
      // Loop-invariant fields of the parameter block live in registers: every inline-asm statement below is a
      // memory barrier to the compiler, so a `c.field` inside the loop is a fresh constant-bank load on the one
      // thread whose latency per k-block sets the pace of the pipeline.
      const int k_blocks = c.k_blocks, k_serp = c.k_serpentine;
      DeviceStatus* const status = c.status;
      const uint32_t wait_us = c.wait_limit_us;
      for (int tile = pair; alive && !c.withhold_loads && tile < pair_tiles; tile += n_pairs, ++it) {
        const TileInfo t = decode_tile(tile);
        for (int kb0 = 0; kb0 < k_blocks; kb0 += KSUB) {
          const int nsub = min(KSUB, k_blocks - kb0);
          if (!ptx::mbar_wait(bar_empty(stage), phase ^ 1u, abort_flag, status, 1, stage, wait_us)) { alive = false; break; }
          const uint32_t leader_full = ptx::mapa(bar_full_b(stage), 0);
          // a half-width tile needs 64 columns of B per CTA: with N-major B that is one of the two
          // 64-column boxes; with K-major B the full 128-row box is fetched and half of it ignored
          const bool half_b = t.bn < BN && B_MN;
          if (leader) ptx::mbar_arrive_expect_tx(bar_full_b(stage), (uint32_t)nsub * (kLeaderBytes - (half_b ? kBHalfBytes : 0)));
          if (kFused) ptx::mbar_arrive_expect_tx(bar_full_a(stage), kABytes);
#pragma unroll
          for (int u = 0; u < KSUB; ++u) {
          if (u >= nsub) break;
          const int kb = kb0 + u, slot = stage * KSUB + u;
          // Every other tile of a CTA walks K backwards.  All pairs are on the same tile count at about the
          // same time, so a wave that starts where the previous one stopped finds the tail of the operand
          // panels it shares with that wave still in L2 (the sum order within a tile changes, the result
          // stays a fixed function of the inputs).
          const int k0 = ((k_serp && (it & 1)) ? k_blocks - 1 - kb : kb) * ((ML & ML_F8) ? 2 * kBK : kBK);   // 128 bytes of K per block
          const uint32_t a_dst = smem_base + SM::off_a + slot * kATileBytes;
          const uint32_t b_dst = smem_base + SM::off_b + slot * kBHalfBytes;
          // A (and the mask): this CTA's 128 rows
          if (kFused) {
            if (A_MN) {
#pragma unroll
              for (int j = 0; j < 2; ++j) ptx::tma_load_3d(a_dst + j * (kBK * 128), &p.tma_a, bar_full_a(stage), t.m0 + 64 * j, k0, t.b);
            } else {
              ptx::tma_load_3d(a_dst, &p.tma_a, bar_full_a(stage), k0, t.m0, t.b);
            }
            if (SM::kHasMask) {
              const uint32_t m_dst = smem_base + SM::off_mask + slot * kATileBytes;
              if (A_MN) {
#pragma unroll
                for (int j = 0; j < 2; ++j) ptx::tma_load_3d(m_dst + j * (kBK * 128), &p.tma_mask, bar_full_a(stage), t.m0 + 64 * j, k0, t.b);
              } else {
                ptx::tma_load_3d(m_dst, &p.tma_mask, bar_full_a(stage), k0, t.m0, t.b);
              }
            }
          } else {
            if (A_MN) {
#pragma unroll
              for (int j = 0; j < 2; ++j) ptx::tma_load_3d_2cta(a_dst + j * (kBK * 128), &p.tma_a, leader_full, t.m0 + 64 * j, k0, t.b);
            } else {
              ptx::tma_load_3d_2cta(a_dst, &p.tma_a, leader_full, k0, t.m0, t.b);
            }
          }
          // B: this CTA's 128 columns of the 256-wide tile
          const int nb0 = t.n0 + (t.bn / 2) * (int)rank;
          if (B_MN) {
            ptx::tma_load_3d_2cta(b_dst, &p.tma_b, leader_full, nb0, k0, t.b);
            if (!half_b) ptx::tma_load_3d_2cta(b_dst + kBK * 128, &p.tma_b, leader_full, nb0 + 64, k0, t.b);
          } else {
            ptx::tma_load_3d_2cta(b_dst, &p.tma_b, leader_full, k0, nb0, t.b);
          }
          }   // u
          if (++stage == GROUPS) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ===================== MMA issuer (leader CTA only) =====================
    if (lane == 0 && leader) {
      const uint32_t idesc_full = (ML & ML_F8) ? ptx::make_idesc_f8(c.f8 & 2 ? 1 : 0, c.f8 & 4 ? 1 : 0, 256, BN)
                                               : ptx::make_idesc_f16(c.ab_format, A_MN ? 1 : 0, B_MN ? 1 : 0, 256, BN);
      const uint32_t idesc_half = (ML & ML_F8) ? ptx::make_idesc_f8(c.f8 & 2 ? 1 : 0, c.f8 & 4 ? 1 : 0, 256, BN / 2)
                                               : ptx::make_idesc_f16(c.ab_format, A_MN ? 1 : 0, B_MN ? 1 : 0, 256, BN / 2);
      constexpr uint32_t a_lbo = A_MN ? kBK * 128 : 16, b_lbo = B_MN ? kBK * 128 : 16;
      constexpr uint32_t a_kadv = A_MN ? 2048 : 32, b_kadv = B_MN ? 2048 : 32;
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool alive = true;
      // parameter-block fields in registers (see the producer)
      const int k_blocks = c.k_blocks, split_from = c.split_count > 0 ? c.split_from : 0x7fffffff;
      DeviceStatus* const status = c.status;
      const uint32_t wait_us = c.wait_limit_us;
      for (int tile = pair; alive && tile < pair_tiles; tile += n_pairs, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
        if (!ptx::mbar_wait(bar_tmem_empty(acc), acc_phase ^ 1u, abort_flag, status, 2, acc, wait_us)) { alive = false; break; }
        ptx::tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        const uint32_t idesc = tile >= split_from ? idesc_half : idesc_full;
        for (int kb0 = 0; kb0 < k_blocks; kb0 += KSUB) {
          const int nsub = min(KSUB, k_blocks - kb0);
          if (!ptx::mbar_wait(bar_full_b(stage), phase, abort_flag, status, 3, stage, wait_us)) { alive = false; break; }
          if (kFused && !ptx::mbar_wait(bar_xform(stage), phase, abort_flag, status, 6, stage, wait_us)) { alive = false; break; }
          ptx::tcgen05_fence_after();
#pragma unroll
          for (int u = 0; u < KSUB; ++u) {
            if (u >= nsub) break;
            const int kb = kb0 + u, slot = stage * KSUB + u;
            const uint32_t a_addr = smem_base + SM::off_a + slot * kATileBytes;
            const uint32_t b_addr = smem_base + SM::off_b + slot * kBHalfBytes;
#pragma unroll
            for (int k = 0; k < kBK / kUmmaK; ++k) {
              const uint64_t adesc = ptx::make_smem_desc_sw128(a_addr + k * a_kadv, a_lbo, 1024);
              const uint64_t bdesc = ptx::make_smem_desc_sw128(b_addr + k * b_kadv, b_lbo, 1024);
              if constexpr ((ML & ML_F8) != 0) ptx::umma_f8_2cta(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
              else ptx::umma_f16_2cta(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
            }
          }
          // free the stage (both of its k-blocks) in both CTAs once these MMAs retire
          ptx::umma_commit_2cta(bar_empty(stage));
          ptx::umma_commit_2cta(ptx::mapa(bar_empty(stage), 1));
          if (++stage == GROUPS) { stage = 0; phase ^= 1u; }
        }
        if (alive) {
          ptx::umma_commit_2cta(bar_tmem_full(acc));
          ptx::umma_commit_2cta(ptx::mapa(bar_tmem_full(acc), 1));
        }
      }
    }
  } else if (warp < kXformWarp0) {
    // ===================== epilogue (both CTAs, own 128 rows x 256 columns) =====================
    EpiEnv env;
    env.core = &c;
    env.scratch = scratch;
    env.bn = BN;
    env.n_epi_threads = NE_WARPS * 32;
    env.epi_warp = warp - 2;
    env.epi_tid = env.epi_warp * 32 + lane;
    env.quadrant = warp & 3;
    int it = 0;
    bool dead = false;
    for (int tile = pair; tile < pair_tiles; tile += n_pairs, ++it) {
      const int acc = it & 1;
      const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
      const TileInfo t = decode_tile(tile);
      const int kColsPerWarp = t.bn / (NE_WARPS / 4);
      const int col_begin = (env.epi_warp / 4) * kColsPerWarp;
      Epi::tile_prepare(p.epi, env, t);   // per-tile staging that does not need the accumulator
      if (!dead && !ptx::mbar_wait(bar_tmem_full(acc), acc_phase, abort_flag, c.status, 4, acc, c.wait_limit_us)) dead = true;
      dead = __any_sync(0xffffffffu, dead);   // the warp decides together (it shares a __syncwarp below)
      typename Epi::State st;
      Epi::tile_begin(p.epi, st);
      if (!dead) {
        ptx::tcgen05_fence_after();
        const int row = env.quadrant * 32 + lane;
        const uint32_t taddr0 = tmem_base + ((uint32_t)(env.quadrant * 32) << 16) + (uint32_t)(acc * BN);
        const int col_end = min(col_begin + kColsPerWarp, ((c.N - t.n0 + CH - 1) / CH) * CH);
        epilogue_walk_chunks<Epi>(p.epi, env, t, st, taddr0, row, col_begin, col_end);
        ptx::tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive_cluster(ptx::mapa(bar_tmem_empty(acc), 0));
      }
      Epi::tile_end(p.epi, env, t, st);
    }
  } else {
    // ===================== mainloop transform (both CTAs, own A tile) =====================
    if (kFused) {
      const int tt = (warp - kXformWarp0) * 32 + lane;
      int stage = 0;
      uint32_t phase = 0;
      bool alive = true;
      for (int tile = pair; alive && tile < pair_tiles; tile += n_pairs) {
        for (int kb = 0; kb < c.k_blocks; ++kb) {
          const bool ok = ptx::mbar_wait(bar_full_a(stage), phase, abort_flag, c.status, 5, stage, c.wait_limit_us);
          if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
          uint4* a = reinterpret_cast<uint4*>(smem + SM::off_a + stage * kATileBytes);
          const uint4* mk = reinterpret_cast<const uint4*>(smem + SM::off_mask + stage * kATileBytes);
          if constexpr ((ML & ML_GENERIC) != 0) {
#pragma unroll 1
            for (int i = 0; i < kATileBytes / 16 / 128; ++i) {
              const int idx = tt + i * 128;
              uint4 va = a[idx];
              uint4 vm;
              if (ML & ML_MASK) vm = mk[idx];
              ml_apply8(c.ml_a, c.ab_format, va, (ML & ML_MASK) ? &vm : nullptr);
              a[idx] = va;
            }
          } else
#pragma unroll
          for (int i = 0; i < kATileBytes / 16 / 128; ++i) {
            const int idx = tt + i * 128;
            uint4 va = a[idx];
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&va);
            if (ML & ML_RELU) {
              const __nv_bfloat162 z = __float2bfloat162_rn(0.0f);
#pragma unroll
              for (int j = 0; j < 4; ++j) h[j] = __hmax2(h[j], z);
            }
            if (ML & ML_MASK) {
              uint4 vm = mk[idx];
              const __nv_bfloat162* hm = reinterpret_cast<const __nv_bfloat162*>(&vm);
#pragma unroll
              for (int j = 0; j < 4; ++j) h[j] = __hmul2(h[j], hm[j]);
            }
            a[idx] = va;
          }
          ptx::fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive_cluster(ptx::mapa(bar_xform(stage), 0));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  }

  // ---- teardown ---------------------------------------------------------------------------------
  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::cluster_sync();   // the peer may still be signalling this CTA's barriers / reading its smem
  if (warp == 1) {
    ptx::tcgen05_fence_after();
    ptx::tmem_dealloc_2cta(tmem_base, kTmemCols);
  }
}

}  // namespace he
