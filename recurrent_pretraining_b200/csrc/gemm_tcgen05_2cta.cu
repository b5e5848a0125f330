// 2-CTA (cta_group::2) variant of the persistent bf16 GEMM: a cluster of two CTAs on neighbouring SMs computes
// one 256 x BN tile.  Each CTA stages its own 128 rows of A and only HALF of the B tile; the pair's tensor cores
// read both halves, so shared-memory fill traffic from L2 per FLOP drops by a third against the 1-CTA 128 x 256
// tile -- the L2 -> SM path, not the tensor pipe, is what limits the 1-CTA kernel on B200.
//
// Protocol (rank 0 of the pair is the leader):
//   * both producers wait on their LOCAL empty barrier and issue their TMA loads with the .cta_group::2 form whose
//     mbarrier operand is the LEADER's full barrier (cluster address from mapa); the leader arms that barrier with
//     the byte count of both CTAs.  No load uses cluster multicast.
//   * only the leader issues tcgen05.mma.cta_group::2 (M = 256); it releases a stage with two tcgen05.commit
//     instructions, one on its own empty barrier and one on the peer's (plain cluster address, no multicast),
//     and publishes a finished accumulator the same way.
//   * each CTA's epilogue warps drain their own 128 TMEM lanes and arrive on the leader's accumulator-empty
//     barrier (the peer through mbarrier.arrive on a cluster address).
// All waits are bounded; a time-out sets the status word and every role falls through to the common exit, where
// the pair synchronises with the cluster barrier before tensor memory is released.
#include <cuda.h>

#include <cstdlib>

#include "common.cuh"
#include "gemm_epilogue.cuh"

namespace b200 {

int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                      uint32_t box_rows, uint32_t box_cols);
int make_tmap_2d_f32(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows);
int num_sms();

constexpr int BM2 = 128;   // rows per CTA (256 per pair)
constexpr int BK2 = 64;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(rank));
  return out;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load into this CTA's smem whose completion bytes are counted on a barrier given by cluster address.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const void* tmap, uint32_t bar_cluster_addr, int x,
                                                 int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma2_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n"
      "  .reg .pred p;\n"
      "  setp.ne.b32 p, %4, 0;\n"
      "  tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive (once the pair's prior MMAs are complete) on one mbarrier given by cluster address
__device__ __forceinline__ void umma2_commit(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr)
               : "memory");
}

// All-gather fused into the GEMM: the B operand (weights [N, K], rows sharded over ranks) is pulled from the owners'
// memory by four extra "copier" warps per CTA into this GPU's full-size buffer, N-tile by N-tile, while the MMA warps
// consume the tiles that have already landed.  Tile order starts at this rank's own shard.  Copiers publish a finished
// N-tile by incrementing done[tile] (release); producers acquire it before their first TMA load of that tile.  All
// TMA loads read LOCAL memory; peers are only touched by plain 16-byte loads.
constexpr int AG_MAX_RANKS = 8;
struct AgParams {
  const __nv_bfloat16* shard[AG_MAX_RANKS];   // shard[q]: rank q's rows [q * rows_per_shard, ...) as [rows, K] contiguous
  __nv_bfloat16* wfull;                       // local [N, ldw] destination, also the TMA source of the GEMM
  int* done;                                  // [tiles_n] counters, zero on entry
  int n_ranks, rank, rows_per_shard, ldw;
};

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_peer_16(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

template <int BN>
struct Smem2 {
  static constexpr int A_BYTES = BM2 * BK2 * 2;        // 16 KB
  static constexpr int B_BYTES = (BN / 2) * BK2 * 2;   // this CTA's half of the B tile
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = 6;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int C_STAGE_OFFSET = BAR_OFFSET + 1024;          // fp32 output modes: 4 warps x 2 x 4 KB
  static constexpr int C_STAGE_BYTES = 4 * 2 * 4096;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + 1024 + 1024;
  static constexpr int TOTAL_F32 = TOTAL + C_STAGE_BYTES;
};

template <int BN, bool A_MN, bool B_MN, int MODE, bool AG = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(AG ? 320 : 192, 1)
gemm2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmA2,
             const __grid_constant__ CUtensorMap tmB, const GemmParams p, const __grid_constant__ AgParams ag,
             const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmC2,
             const __grid_constant__ CUtensorMap tmC3) {
  using L = Smem2<BN>;
  constexpr int STAGES = L::STAGES;
  constexpr int ACC_STRIDE = 256;
  constexpr int BNH = BN / 2;
  constexpr uint32_t IDESC = make_idesc_bf16(2 * BM2, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
  // SwiGLU: the pair's 256 accumulator columns are [128 gate | 128 up] of the same 128 output columns; CTA 0 stages
  // the gate rows of B, CTA 1 the up rows (p.swiglu_n rows further down), and p.N is the OUTPUT width.
  constexpr int BN_OUT = is_swiglu(MODE) ? BN / 2 : BN;
  static_assert(!is_swiglu(MODE) || (BN == 256 && !A_MN && !B_MN), "SwiGLU epilogue: NT GEMM with 256-wide MMA tiles");
  static_assert(!B_MN || (BNH % 64 == 0), "MN-major B needs 64-column chunks per CTA");

  extern __shared__ uint8_t smem_raw[];
  // identical offsets in both CTAs of the pair (the MMA descriptors are shared)
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * L::STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;   // [2]
  uint64_t* tempty_bar = tfull_bar + 2;       // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;

  const int tiles_m = (p.M + 2 * BM2 - 1) / (2 * BM2);
  const int tiles_n = (p.N + BN_OUT - 1) / BN_OUT;
  const int num_tiles = tiles_m * tiles_n;
  const int nk1 = (p.K1 + BK2 - 1) / BK2;
  const int nk2 = (p.K2 + BK2 - 1) / BK2;
  const int nk = nk1 + nk2;
  // N-tile of a linear tile index; with the fused all-gather the order is rotated to start at this rank's shard
  const int ag_first = AG ? (ag.rank * ag.rows_per_shard) / BN : 0;
  // (m tile, n tile) of a linear index: grouped raster, except that the fused all-gather walks whole n tiles in shard
  // order (its counters are per n tile)
  auto tile_mn = [&](int tile, int& mi, int& ni) {
    if constexpr (AG) {
      mi = tile % tiles_m;
      ni = (ag_first + tile / tiles_m) % tiles_n;
    } else {
      tile_coords(tile, tiles_m, tiles_n, p.raster, mi, ni);
    }
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 8);   // 4 epilogue warps of each CTA
    }
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc2(tmem_slot, 512);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // both CTAs' barriers exist before any remote arrive or remote complete_tx
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer (both CTAs)
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      if (nk2 > 0) tma_prefetch_desc(&tmA2);
      // stage index and phase advance by increment (no division in the per-k-block path of this single thread)
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      const uint32_t fb0 = mapa_shared(smem_u32(&full_bar[0]), 0);   // leader's full barriers: fb0 + 8 * stage
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
        int mt, nt;
        tile_mn(tile, mt, nt);
        const int m0 = mt * (2 * BM2) + static_cast<int>(rank) * BM2;
        const int n0 = is_swiglu(MODE) ? nt * BN_OUT + static_cast<int>(rank) * p.swiglu_n
                                            : nt * BN + static_cast<int>(rank) * BNH;
        if constexpr (AG) {
          // the weight rows of this N-tile must have landed in the local buffer (every CTA's copiers add one)
          const unsigned long long t0 = globaltimer_ns();
          while (ld_acquire_gpu(ag.done + nt) < static_cast<int>(gridDim.x)) {
            if (*abort_flag || globaltimer_ns() - t0 > WAIT_LIMIT_NS) {
              *abort_flag = 1;
              if (p.err) atomicCAS(p.err, 0, ERR_WAIT_PEER_FLAG);
              ok = false;
              break;
            }
            __nanosleep(64);
          }
          if (!ok) break;
          asm volatile("fence.proxy.async;" ::: "memory");   // generic-proxy writes of the copiers -> TMA reads
        }
        for (int kb = 0; kb < nk; ++kb) {
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.err, ERR_WAIT_STAGE_EMPTY)) { ok = false; break; }
          uint8_t* sa = smem + s * L::STAGE_BYTES;
          uint8_t* sb = sa + L::A_BYTES;
          if (leader) mbar_expect_tx(&full_bar[s], 2 * L::STAGE_BYTES);
          const uint32_t fb = fb0 + 8u * s;
          const bool second = kb >= nk1;
          const int ka = (second ? (kb - nk1) : kb) * BK2;
          const int kbcol = second ? (p.K1 + ka) : ka;
          if constexpr (!A_MN) {
            if (second) tma_load_2d_pair(sa, &tmA2, fb, ka, m0);
            else tma_load_2d_pair(sa, &tmA, fb, ka, m0);
          } else {
#pragma unroll
            for (int c = 0; c < BM2 / 64; ++c) tma_load_2d_pair(sa + c * (BK2 * 128), &tmA, fb, m0 + c * 64, ka);
          }
          if constexpr (!B_MN) {
            tma_load_2d_pair(sb, &tmB, fb, kbcol, n0);
          } else {
#pragma unroll
            for (int c = 0; c < BNH / 64; ++c) tma_load_2d_pair(sb + c * (BK2 * 128), &tmB, fb, n0 + c * 64, kbcol);
          }
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && leader) {
      uint32_t tcount = 0;
      bool ok = true;
      // The tensor pipe needs a new MMA every ~120 cycles; this single thread must not spend longer than that per
      // instruction, so stage, phase, shared-memory descriptors and barrier addresses all advance by increments.
      int s = 0;
      uint32_t ph = 0;
      const uint32_t smem0 = smem_u32(smem);
      const uint64_t desc_hi_a = A_MN ? make_smem_desc(0, BK2 * 128, 1024) : make_smem_desc(0, 16, 1024);
      const uint64_t desc_hi_b = B_MN ? make_smem_desc(0, BK2 * 128, 1024) : make_smem_desc(0, 16, 1024);
      constexpr uint32_t KSTEP_A = (A_MN ? 2048 : 32) >> 4, KSTEP_B = (B_MN ? 2048 : 32) >> 4;
      const uint32_t eb0 = mapa_shared(smem_u32(&empty_bar[0]), 0), eb1 = mapa_shared(smem_u32(&empty_bar[0]), 1);
      const uint32_t tb0 = mapa_shared(smem_u32(&tfull_bar[0]), 0), tb1 = mapa_shared(smem_u32(&tfull_bar[0]), 1);
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters, ++tcount) {
        const int acc = tcount & 1;
        const uint32_t aph = (tcount >> 1) & 1;
        if (!mbar_wait(&tempty_bar[acc], aph ^ 1, abort_flag, p.err, ERR_WAIT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * ACC_STRIDE;
        for (int kb = 0; kb < nk; ++kb) {
          if (!mbar_wait(&full_bar[s], ph, abort_flag, p.err, ERR_WAIT_TMA_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem0 + s * L::STAGE_BYTES;
          uint64_t adesc = desc_hi_a | ((sa & 0x3FFFF) >> 4);
          uint64_t bdesc = desc_hi_b | (((sa + L::A_BYTES) & 0x3FFFF) >> 4);
#pragma unroll
          for (int k = 0; k < BK2 / 16; ++k) {
            umma2_bf16(d_tmem, adesc, bdesc, IDESC, (kb | k) ? 1u : 0u);
            adesc += KSTEP_A;   // the start-address field sits in the low bits: stepping it is a plain add
            bdesc += KSTEP_B;
          }
          umma2_commit(eb0 + 8u * s);
          umma2_commit(eb1 + 8u * s);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (ok) {
          umma2_commit(tb0 + 8u * acc);
          umma2_commit(tb1 + 8u * acc);
        }
      }
    }
  } else if (AG && warp >= 6) {
    // ------------------------------------------------------------------ copiers (warps 6..9 of every CTA)
    if constexpr (AG) {
      const int ct = threadIdx.x - 192;                       // 0..127
      const size_t g = static_cast<size_t>(blockIdx.x) * 128 + ct, gstride = static_cast<size_t>(gridDim.x) * 128;
      const int vec_per_row = (p.K1 + p.K2) >> 3;             // 16-byte vectors per weight row
      for (int i = 0; i < tiles_n; ++i) {
        const int nt = (ag_first + i) % tiles_n;
        const int r0 = nt * BN, r1 = min(p.N, r0 + BN);
        const size_t nvec = static_cast<size_t>(r1 - r0) * vec_per_row;
        // AG_DEPTH independent 16-byte peer loads per thread are in flight before the first store: a peer load takes
        // microseconds, and the bytes in flight (threads x depth x 16) must cover latency x link bandwidth
        constexpr int AG_DEPTH = 12;
        for (size_t v = g; v < nvec; v += AG_DEPTH * gstride) {
          uint4 buf[AG_DEPTH];
#pragma unroll
          for (int u = 0; u < AG_DEPTH; ++u) {
            const size_t idx = v + u * gstride;
            if (idx < nvec) {
              const int row = r0 + static_cast<int>(idx / vec_per_row), col = static_cast<int>(idx % vec_per_row);
              const int owner = min(row / ag.rows_per_shard, ag.n_ranks - 1);
              const __nv_bfloat16* src = ag.shard[owner] + static_cast<size_t>(row - owner * ag.rows_per_shard) * (vec_per_row * 8);
              buf[u] = ld_peer_16(reinterpret_cast<const uint4*>(src) + col);
            }
          }
#pragma unroll
          for (int u = 0; u < AG_DEPTH; ++u) {
            const size_t idx = v + u * gstride;
            if (idx < nvec) {
              const int row = r0 + static_cast<int>(idx / vec_per_row), col = static_cast<int>(idx % vec_per_row);
              reinterpret_cast<uint4*>(ag.wfull + static_cast<size_t>(row) * ag.ldw)[col] = buf[u];
            }
          }
        }
        named_barrier_sync(2, 128);
        if (ct == 0) {
          __threadfence();
          atomicAdd(ag.done + nt, 1);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (both CTAs, warps 2..5)
    const int quad = warp & 3;
    uint32_t tcount = 0;
    constexpr bool F32_MODE = MODE == OUT_F32 || MODE == OUT_F32_ACC;
    // modes with a shared-memory staged epilogue
    constexpr bool STAGED = (F32_MODE || MODE == OUT_BF16 || MODE == OUT_BF16_ROPE || MODE == OUT_SWIGLU ||
                             MODE == OUT_SWIGLU_SAVE || MODE == OUT_DSWIGLU) && !AG;
    uint8_t* c_stage = smem + L::C_STAGE_OFFSET + quad * 8192;   // only backed by memory in the fp32 output modes
    int c_buf = 0;
    for (int tile = cluster_id; tile < num_tiles; tile += num_clusters, ++tcount) {
      const int acc = tcount & 1;
      const uint32_t aph = (tcount >> 1) & 1;
      int mt, nt;
      tile_mn(tile, mt, nt);
      const int m0 = mt * (2 * BM2) + static_cast<int>(rank) * BM2;
      const int n0 = nt * BN_OUT;
      if (!mbar_wait(&tfull_bar[acc], aph, abort_flag, p.err, ERR_WAIT_TMEM_FULL)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * ACC_STRIDE + (static_cast<uint32_t>(quad * 32) << 16);
      if constexpr (F32_MODE) {
        if (p.tma_c) epilogue_tile_tma_f32<BN_OUT, MODE>(p, &tmC, taddr, m0 + quad * 32, n0, c_stage, lane, c_buf);
        else epilogue_tile<BN_OUT, MODE>(p, taddr, m0 + quad * 32 + lane, n0);
      } else if constexpr (STAGED) {
        if (!p.tma_c) epilogue_tile<BN_OUT, MODE>(p, taddr, m0 + quad * 32 + lane, n0);
        else if constexpr (MODE == OUT_BF16_ROPE)
          epilogue_tile_tma_rope<BN_OUT>(p, &tmC, taddr, m0 + quad * 32, n0, c_stage, lane, c_buf);
        else if constexpr (MODE == OUT_SWIGLU)
          epilogue_tile_tma_swiglu<BN_OUT>(p, &tmC, taddr, m0 + quad * 32, n0, c_stage, lane, c_buf);
        else if constexpr (MODE == OUT_SWIGLU_SAVE)
          epilogue_tile_tma_swiglu_save<BN_OUT>(p, &tmC, &tmC2, &tmC3, taddr, m0 + quad * 32, n0, c_stage, lane, c_buf);
        else if constexpr (MODE == OUT_DSWIGLU)
          epilogue_tile_tma_dswiglu<BN_OUT>(p, &tmC, &tmC2, taddr, m0 + quad * 32, n0, c_stage, lane, c_buf);
        else epilogue_tile_tma_bf16<BN_OUT>(p, &tmC, taddr, m0 + quad * 32, n0, c_stage, lane, c_buf);
      } else {
        epilogue_tile<BN_OUT, MODE>(p, taddr, m0 + quad * 32 + lane, n0);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&tempty_bar[acc]), 0));
    }
    if constexpr (STAGED) {
      if (p.tma_c && lane == 0) bulk_wait_all();   // this lane's stores / reductions have reached memory
    }
  }

  // common exit: nobody leaves (and no tensor memory is released) while the partner may still touch this CTA
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc2(tmem_base, 512);
  }
}

template <int BN, bool A_MN, bool B_MN, int MODE, bool AG = false>
static int launch2(const CUtensorMap& ta, const CUtensorMap& ta2, const CUtensorMap& tb, const GemmParams& p,
                   cudaStream_t stream, int max_ctas, const AgParams* agp = nullptr, const CUtensorMap* tcp = nullptr,
                   const CUtensorMap* tcp2 = nullptr, const CUtensorMap* tcp3 = nullptr) {
  using L = Smem2<BN>;
  auto kern = gemm2_kernel<BN, A_MN, B_MN, MODE, AG>;
  constexpr int SMEM = ((MODE == OUT_F32 || MODE == OUT_F32_ACC || MODE == OUT_BF16 || MODE == OUT_BF16_ROPE ||
                         MODE == OUT_SWIGLU || MODE == OUT_SWIGLU_SAVE || MODE == OUT_DSWIGLU) && !AG)
                            ? L::TOTAL_F32 : L::TOTAL;
  static int max_clusters = -1;
  if (max_clusters < 0) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) return -10;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(num_sms() & ~1, 1, 1);
    cfg.blockDim = dim3(AG ? 320 : 192, 1, 1);
    cfg.dynamicSmemBytes = SMEM;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) n = num_sms() / 2;
    max_clusters = n;
  }
  constexpr int BN_OUT = is_swiglu(MODE) ? BN / 2 : BN;
  const int tiles = ((p.M + 2 * BM2 - 1) / (2 * BM2)) * ((p.N + BN_OUT - 1) / BN_OUT);
  int clusters = tiles < max_clusters ? tiles : max_clusters;
  if (max_ctas > 0 && clusters > max_ctas / 2) clusters = max_ctas / 2;
  if (clusters <= 0) return 0;
  AgParams ag = {};
  if (agp) ag = *agp;
  GemmParams pp = p;
  if (!tcp) pp.tma_c = 0;
  kern<<<2 * clusters, AG ? 320 : 192, SMEM, stream>>>(ta, ta2, tb, pp, ag, tcp ? *tcp : ta, tcp2 ? *tcp2 : ta,
                                                       tcp3 ? *tcp3 : ta);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Entry used by b200_gemm: returns -100 when the 2-CTA kernel does not cover the request.
int gemm_2cta_dispatch(const void* A, const void* A2, const void* B, const GemmParams& p, int lda, int lda2, int ldb,
                       int a_mn, int b_mn, int out_mode, int bn, int max_ctas, cudaStream_t st) {
  if (is_swiglu(out_mode) && (a_mn || b_mn || bn != 256 || p.K2 > 0)) return -100;
  if (bn == 240 && (a_mn || b_mn)) return -100;   // the 240-wide instantiation is NT only
  if (bn != 256 && bn != 240) return -100;
  const int K = p.K1 + p.K2;
  CUtensorMap ta, ta2, tb;
  int rc;
  if (!a_mn) rc = make_tmap_2d_bf16(&ta, A, p.M, p.K1, lda, BM2, BK2);
  else rc = make_tmap_2d_bf16(&ta, A, p.K1, p.M, lda, BK2, 64);
  if (rc) return rc;
  ta2 = ta;
  if (p.K2 > 0) {
    rc = make_tmap_2d_bf16(&ta2, A2, p.M, p.K2, lda2, BM2, BK2);
    if (rc) return rc;
  }
  const int brows = is_swiglu(out_mode) ? 2 * p.N : p.N;
  if (!b_mn) rc = make_tmap_2d_bf16(&tb, B, brows, K, ldb, bn / 2, BK2);
  else rc = make_tmap_2d_bf16(&tb, B, K, p.N, ldb, BK2, 64);
  if (rc) return rc;

  // fp32 output of 256-wide tiles leaves through bulk tensor stores / reductions when C can be described by a tensor
  // map (16-byte aligned base and row pitch); B200_GEMM_TMA_C=0 keeps the per-thread epilogue
  CUtensorMap tc;
  const CUtensorMap* tcp = nullptr;
  GemmParams pc = p;
  pc.tma_c = 0;
  static const bool tma_c_on = [] { const char* e = getenv("B200_GEMM_TMA_C"); return !(e && e[0] == '0'); }();
  if ((out_mode == OUT_F32 || out_mode == OUT_F32_ACC) && bn == 256 && tma_c_on &&
      make_tmap_2d_f32(&tc, p.C, p.M, p.N, p.ldc, 32) == 0) {
    tcp = &tc;
    pc.tma_c = 1;
  }
  static const bool tma_c16_on = [] { const char* e = getenv("B200_GEMM_TMA_C16"); return !(e && e[0] == '0'); }();
  if ((out_mode == OUT_BF16 || out_mode == OUT_BF16_ROPE || out_mode == OUT_SWIGLU) && tma_c_on && tma_c16_on &&
      make_tmap_2d_bf16(&tc, p.C, p.M, p.N, p.ldc, 32, 64) == 0) {
    tcp = &tc;
    pc.tma_c = 1;
  }
  // SwiGLU with stored pre-activation: y [M, I] plus the gate and up halves of h [M, 2 I]; dSwiGLU: the dg and du
  // halves of the [M, 2 I] output.  Each half is a tensor of its own (clipping at its right edge).
  CUtensorMap tc2, tc3;
  const CUtensorMap *tcp2 = nullptr, *tcp3 = nullptr;
  static const bool tma_h_on = [] { const char* e = getenv("B200_GEMM_TMA_H"); return !(e && e[0] == '0'); }();
  if (tma_c_on && tma_c16_on && tma_h_on && bn == 256 && (p.swiglu_n & 7) == 0) {
    const __nv_bfloat16* h = p.resid;
    if (out_mode == OUT_SWIGLU_SAVE && h &&
        make_tmap_2d_bf16(&tc, p.C, p.M, p.N, p.ldc, 32, 64) == 0 &&
        make_tmap_2d_bf16(&tc2, h, p.M, p.N, p.ld_resid, 32, 64) == 0 &&
        make_tmap_2d_bf16(&tc3, h + p.swiglu_n, p.M, p.N, p.ld_resid, 32, 64) == 0) {
      tcp = &tc; tcp2 = &tc2; tcp3 = &tc3;
      pc.tma_c = 1;
    }
    if (out_mode == OUT_DSWIGLU && h && (reinterpret_cast<uintptr_t>(h) & 15) == 0 && (p.ld_resid & 7) == 0 &&
        make_tmap_2d_bf16(&tc, p.C, p.M, p.N, p.ldc, 32, 64) == 0 &&
        make_tmap_2d_bf16(&tc2, reinterpret_cast<const __nv_bfloat16*>(p.C) + p.swiglu_n, p.M, p.N, p.ldc, 32, 64) == 0) {
      tcp = &tc; tcp2 = &tc2;
      pc.tma_c = 1;
    }
  }
#define DISPATCH2(BN_, AMN_, BMN_)                                                                  \
  switch (out_mode) {                                                                               \
    case OUT_BF16: return launch2<BN_, AMN_, BMN_, OUT_BF16>(ta, ta2, tb, pc, st, max_ctas, nullptr, tcp);       \
    case OUT_F32: return launch2<BN_, AMN_, BMN_, OUT_F32>(ta, ta2, tb, pc, st, max_ctas, nullptr, tcp);         \
    case OUT_F32_ACC: return launch2<BN_, AMN_, BMN_, OUT_F32_ACC>(ta, ta2, tb, pc, st, max_ctas, nullptr, tcp); \
    case OUT_BF16_RESID: return launch2<BN_, AMN_, BMN_, OUT_BF16_RESID>(ta, ta2, tb, p, st, max_ctas); \
    default: return -100;                                                                           \
  }
  if (out_mode == OUT_SWIGLU) return launch2<256, false, false, OUT_SWIGLU>(ta, ta2, tb, pc, st, max_ctas, nullptr, tcp);
  if (out_mode == OUT_SWIGLU_SAVE)
    return launch2<256, false, false, OUT_SWIGLU_SAVE>(ta, ta2, tb, pc, st, max_ctas, nullptr, tcp, tcp2, tcp3);
  if (out_mode == OUT_BF16_LSE) {
    if (a_mn || b_mn || bn != 256) return -100;
    return launch2<256, false, false, OUT_BF16_LSE>(ta, ta2, tb, p, st, max_ctas);
  }
  if (out_mode == OUT_DSWIGLU) {
    if (a_mn || !b_mn || bn != 256) return -100;
    return launch2<256, false, true, OUT_DSWIGLU>(ta, ta2, tb, pc, st, max_ctas, nullptr, tcp, tcp2);
  }
  if (out_mode == OUT_BF16_ROPE) {
    if (a_mn || b_mn) return -100;
    if (bn == 240) return launch2<240, false, false, OUT_BF16_ROPE>(ta, ta2, tb, pc, st, max_ctas, nullptr, tcp);
    return launch2<256, false, false, OUT_BF16_ROPE>(ta, ta2, tb, pc, st, max_ctas, nullptr, tcp);
  }
  if (!a_mn && !b_mn) {
    if (bn == 256) { DISPATCH2(256, false, false) }
    if (bn == 240) { DISPATCH2(240, false, false) }
  } else if (!a_mn && b_mn) {
    DISPATCH2(256, false, true)
  } else if (a_mn && b_mn) {
    DISPATCH2(256, true, true)
  } else {
    DISPATCH2(256, true, false)
  }
#undef DISPATCH2
  return -100;
}

}  // namespace b200

using namespace b200;

// C[M, N] (bf16) = A[M, K] Wfull[N, K]^T where W's rows are sharded over `n_ranks` GPUs: shard_ptrs[q] is rank q's
// [rows_per_shard, K] block (peer-mapped), wfull the local [N, K] buffer that the kernel fills while it multiplies
// (afterwards it holds the gathered weight for the remaining uses in this step).  `done`: int[ceil(N / bn)], zeroed by
// this call.  bn: 240 or 256 (0 picks).
extern "C" __attribute__((visibility("default"))) int b200_ag_gemm(
    const void* A, void* const* shard_ptrs, void* wfull, void* C, int* done, int M, int N, int K, int lda, int ldc,
    int n_ranks, int rank, int rows_per_shard, int bn, void* stream, int* err) {
  if (n_ranks < 1 || n_ranks > AG_MAX_RANKS || (K & 7) || M < 256) return -1;
  if (bn == 0) bn = (N % 256 != 0 && N % 240 == 0) ? 240 : 256;
  if (bn != 240 && bn != 256) return -1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int tiles_n = (N + bn - 1) / bn;
  if (cudaMemsetAsync(done, 0, sizeof(int) * tiles_n, st) != cudaSuccess) return -2;
  GemmParams p = {};
  p.M = M; p.N = N; p.K1 = K; p.K2 = 0; p.ldc = ldc; p.ld_resid = 0; p.swiglu_n = N; p.ksplit = 1;
  p.C = C; p.resid = nullptr; p.err = err;
  AgParams ag = {};
  for (int q = 0; q < n_ranks; ++q) ag.shard[q] = reinterpret_cast<const __nv_bfloat16*>(shard_ptrs[q]);
  ag.wfull = reinterpret_cast<__nv_bfloat16*>(wfull);
  ag.done = done; ag.n_ranks = n_ranks; ag.rank = rank; ag.rows_per_shard = rows_per_shard; ag.ldw = K;
  CUtensorMap ta, tb;
  int rc = make_tmap_2d_bf16(&ta, A, M, K, lda, BM2, BK2);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tb, wfull, N, K, K, bn / 2, BK2);
  if (rc) return rc;
  if (bn == 240) return launch2<240, false, false, OUT_BF16, true>(ta, ta, tb, p, st, 0, &ag);
  return launch2<256, false, false, OUT_BF16, true>(ta, ta, tb, p, st, 0, &ag);
}
