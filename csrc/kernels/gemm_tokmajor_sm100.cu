// Token-major tcgen05 GEMM for block-scaled e4m3 operands (sm_100a).
//
//   out[t, n] = sum_k X[t, k] * W[g, n, k]            (t in group g's row segment)
//
// Same math and argument conventions as the weight-stationary kernel in gemm_sm100.cu, opposite orientation:
// the 128 token rows of a tile are the UMMA M dimension (one token per TMEM lane and per epilogue thread), 256
// weight rows are the UMMA N dimension (at N = 256 a tcgen05.mma computes for longer than it takes to issue,
// so the tensor pipe stays busy even though every 128-wide K block needs its own hand-shake).  With DeepSeek-style scales (one activation scale per token and
// 128-wide K block, one weight scale per 128x128 block) every 128-wide K block has to be promoted from TMEM
// into fp32 registers with its own multiplier.  In this orientation that multiplier is a single scalar per
// thread and K block (its token's activation scale times the tile's weight scale).  With the weights on the
// lanes every thread needs the activation scales of all its token columns in registers instead, 64 KB per K
// block and SM through the shared-memory return path, which alone takes longer than the MMAs.
//
// The output row of a thread is contiguous in memory, so the epilogue writes 16-byte vectors.
//
// One persistent CTA per SM:
//   warp 0       TMA producer (one lane)
//   warp 1       MMA issue (one elected lane)
//   warps 2..3   idle (they only take part in the register hand-over)
//   warps 4..11  epilogue: two groups of four warps, each group owns 64 of the 128 output columns
// The four control warps give most of their registers to the epilogue warps (setmaxnreg), which hold the
// promoted accumulators, 128 fp32 per thread.
//
// The 256 weight rows of a tile are two blocks of 128 (each with its own weight scale).  EPI 0 = store: the
// blocks are consecutive output features (bf16 or fp32 output, optional per-row multiplier).  EPI 1 / 2 =
// SwiGLU: W holds n_out gate rows, then n_out up rows, per group; block 0 is 128 gate rows, block 1 the
// matching up rows, and the tile produces 128 output features: EPI 1 -> bf16, EPI 2 -> e4m3 with one scale
// per token and 128 output features (exactly one tile).
//
// KIND 0 = bf16 operands: the whole K range accumulates in TMEM and the epilogue runs once per tile.
// KIND 1 = e4m3 operands with block scales, promoted per K block as described above.
//
// Fused collectives (tensor-parallel attention), both over peer memory mapped into this process:
//   * reduce-scatter epilogue: this rank's GEMM result is a partial sum; token row t belongs to rank
//     t / rows_per_rank, and the epilogue writes each row straight into that rank's receive slab
//     [source rank][local row][n_out] with 16-byte peer stores, tile by tile while later tiles still compute.
//     The last CTA publishes one flag per destination (release at system scope); tp_fused.cu sums the slabs.
//   * all-gather prologue: X is a gather buffer that every rank fills with its own row block; the producer
//     waits (bounded) for the flag of the source rank of a tile's rows before it issues the tile's first TMA
//     load, and takes this rank's own rows first, so the GEMM starts before the remote rows have arrived.
// Stands where the reference runs o_proj then reduce_scatter, and all_gather then the q_a / MLP input
// projections (omni/models/common/layers/attention/deepseek_mla.py:437-470,
// omni/models/common/layers/linear.py:139-199).
//
// Stands where the reference calls npu_quant_matmul / npu_grouped_matmul / npu_dequant_swiglu_quant
// (omni/models/common/layers/moe/fused_moe/fused_moe.py:541-575,
//  omni/quantization/compressed_tensors/compressed_tensors_moe.py:221-253).
#include "../include/omni_ptx.cuh"
#include "../include/tma_host.h"

namespace omni {

struct TmGemmParams {
  int G;                 // groups (experts); 1 for a dense GEMM
  int n_out;             // output features per group and accumulator
  int K;
  int T;                 // rows when seg_* are null
  const int* seg_start;  // [G] first row of the group's segment in X/out, or null
  const int* seg_len;    // [G] rows in the segment, or null
  int w_rows_per_group;  // n_out (store) or 2 * n_out (SwiGLU)
  const float* w_scale;  // [G, w_rows_per_group/128, K/128]
  const float* x_scale;  // [K/128, x_scale_ld]
  int x_scale_ld;
  void* out;
  int out_ld;
  int out_f32;
  float* out_scale;      // EPI 2: [n_out/128, out_scale_ld]
  int out_scale_ld;
  const float* row_scale;  // optional [rows]
  int x_group_col;       // head-batched mode: group g reads X columns [g*x_group_col, +K) ...
  int out_group_col;     // ... and writes out columns [g*out_group_col, +n_out)
  // reduce-scatter epilogue (rs_world > 1): out is ignored, rows go to rs_out[row / rs_rows_per_rank]
  int rs_world, rs_rank, rs_rows_per_rank;
  void* rs_out[8];       // per destination rank: slab base [world][rows_per_rank][out_ld] (bf16)
  int* rs_flag[8];       // per destination rank: flag word of this source rank
  int* rs_done;          // local: CTAs finished (reset by the last one)
  int* rs_epoch;         // local: round counter, advanced by the last CTA and published to the destinations
  // all-gather prologue (ag_world > 1): rows [s*ag_rows_per_rank, +ag_rows_per_rank) of X arrive from rank s
  int ag_world, ag_rank, ag_rows_per_rank;
  const int* ag_flag;    // local: [world] round of the last block received from each rank
  const int* ag_epoch;   // local: current round (advanced by the push kernel that precedes this launch)
  unsigned long long ag_wait_ns;
  OmniStatus* status;
};

constexpr int TM_THREADS = 384;
constexpr int TM_REGS_BASE = 168;   // 65536 / 384, rounded down to a multiple of 8: what every thread starts with
constexpr int TM_REGS_CTRL = 64, TM_REGS_EPI = 216;
// The raise in the epilogue groups blocks in hardware until the control group has released enough registers,
// so the budget must balance or the kernel never gets past that instruction.
static_assert(128 * (TM_REGS_BASE - TM_REGS_CTRL) >= 256 * (TM_REGS_EPI - TM_REGS_BASE),
              "setmaxnreg: the control warps release fewer registers than the epilogue warps request");
constexpr int TM_MAX_GROUPS = 1024;
constexpr int TM_BN = 128;          // weight rows per block; a tile has two blocks (UMMA N = 256)
constexpr int TM_CW = 64;           // output columns per epilogue group

struct TmSmem {
  static constexpr int A_BYTES = 128 * 128;            // 128 tokens x 128 B
  static constexpr int B_BYTES = TM_BN * 128;          // one block of 128 weight rows
  static constexpr int STAGE_BYTES = A_BYTES + 2 * B_BYTES;
  static constexpr int MAX_STAGES = 8;
  static constexpr int SC_BYTES = MAX_STAGES * 128 * 4;      // activation-scale ring, one float per token and stage
  static constexpr int PREFIX_BYTES = (TM_MAX_GROUPS + 4) * 4;
  static constexpr int AUX_BYTES = 1024 /*barriers*/ + PREFIX_BYTES + 1024 /*amax exchange*/ + SC_BYTES;
  static constexpr int STAGES_RAW = (225 * 1024 - AUX_BYTES - 1024) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > MAX_STAGES ? MAX_STAGES : STAGES_RAW;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + AUX_BYTES + 1024;
};

enum { TMS_PROD_EMPTY = 21, TMS_MMA_FULL = 22, TMS_MMA_TMEM_EMPTY = 23, TMS_EPI_TMEM_FULL = 24, TMS_TMEM_BASE = 25,
       TMS_AG_FLAG = 26 };

__device__ __forceinline__ void tm_bulk_load_1d(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tm_fma2(float2& acc, float2 a, float2 b) {
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(reinterpret_cast<uint64_t&>(acc))
      : "l"(reinterpret_cast<uint64_t&>(a)), "l"(reinterpret_cast<uint64_t&>(b)));
}


template <int KIND, int EPI>
__global__ void __launch_bounds__(TM_THREADS, 1)
gemm_tokmajor_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                     const TmGemmParams p) {
  using L = TmSmem;
  constexpr int STAGES = L::STAGES;
  constexpr bool GLU = EPI != 0;
  constexpr int BK_ELEMS = (KIND == 0) ? 64 : 128;   // one 128-byte swizzle span
  constexpr int NB = 2;                          // weight-row blocks per tile
  constexpr int ACC_COLS = NB * TM_BN;           // TMEM columns of one accumulator buffer
  constexpr int NBUF = 512 / ACC_COLS;
  constexpr uint32_t tmem_base = 0;              // the whole TMEM is allocated, so the base is column 0

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* aux = smem + STAGES * L::STAGE_BYTES;
  uint64_t* full_bar = (uint64_t*)aux;                   // [STAGES]
  uint64_t* empty_bar = full_bar + L::MAX_STAGES;        // [STAGES]
  uint64_t* tfull_bar = empty_bar + L::MAX_STAGES;       // [NBUF]
  uint64_t* tempty_bar = tfull_bar + 4;                  // [NBUF]
  uint32_t* tmem_slot = (uint32_t*)(tempty_bar + 4);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  int* epi_counter = (int*)(tmem_slot + 2);              // rendezvous of the eight epilogue warps (only grows)
  int* tile_prefix = (int*)(aux + 1024);                 // [G + 1]
  float* amax_x = (float*)(aux + 1024 + L::PREFIX_BYTES);  // [2 groups][128 rows]
  float* sc_ring = amax_x + 256;                         // [STAGES][128], 16-byte aligned (bulk copies)
  static_assert((1024 + L::PREFIX_BYTES + 1024) % 16 == 0, "scale ring must be 16-byte aligned");

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb = (p.K + BK_ELEMS - 1) / BK_ELEMS;
  const int n_tiles = GLU ? p.n_out / TM_BN : (p.n_out + 2 * TM_BN - 1) / (2 * TM_BN);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      // fp8: released by the eight epilogue warps once they have read the stage's scale slot, which they only
      // do after the stage's MMAs have retired (they waited for tfull).  bf16: released by the MMA commit.
      mbar_init(&empty_bar[s], KIND == 1 ? 8 : 1);
    }
    for (int b = 0; b < NBUF; ++b) {
      mbar_init(&tfull_bar[b], 1);
      mbar_init(&tempty_bar[b], 8);
    }
    *abort_flag = 0;
    *epi_counter = 0;
    mbar_fence_init();
    // tiles per group: ceil(len / 128) token tiles x n_tiles, token tile fastest (neighbouring CTAs then read
    // the same weight tile at about the same time)
    int acc = 0;
    for (int g = 0; g < p.G; ++g) {
      tile_prefix[g] = acc;
      const int len = p.seg_len ? p.seg_len[g] : p.T;
      acc += ((len + 127) / 128) * n_tiles;
    }
    tile_prefix[p.G] = acc;
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  if (*tmem_slot != 0u) {   // cannot happen while the whole TMEM is requested; never compute on a wrong base
    if (threadIdx.x == 0) { *abort_flag = 1; report_status(p.status, OMNI_ERR_MBAR_TIMEOUT, TMS_TMEM_BASE, (int)*tmem_slot); }
    __syncthreads();
    if (warp == 1) tmem_dealloc(*tmem_slot, 512);
    return;
  }
  const int total_tiles = tile_prefix[p.G];

  // tile index -> (group, weight tile, first row, rows valid)
  auto decode_tile = [&](int tile, int& g, int& nt, int& row0, int& rows) {
    int lo = 0, hi = p.G - 1;
    while (lo < hi) {  // last g with tile_prefix[g] <= tile
      const int mid = (lo + hi + 1) >> 1;
      if (tile_prefix[mid] <= tile) lo = mid; else hi = mid - 1;
    }
    g = lo;
    const int local = tile - tile_prefix[g];
    const int len = p.seg_len ? p.seg_len[g] : p.T;
    const int m_tiles = (len + 127) / 128;
    nt = local / m_tiles;
    int mt = local - nt * m_tiles;
    if (p.ag_world > 1 && p.ag_rows_per_rank >= 128) {          // own rows first: they need no wait
      mt += p.ag_rank * (p.ag_rows_per_rank / 128);
      if (mt >= m_tiles) mt -= m_tiles;
    } else if (p.rs_world > 1 && p.rs_rows_per_rank >= 128) {   // own rows last: remote rows have further to go
      mt += (p.rs_rank + 1) * (p.rs_rows_per_rank / 128);
      if (mt >= m_tiles) mt -= m_tiles;
    }
    const int start = p.seg_start ? p.seg_start[g] : 0;
    row0 = start + mt * 128;
    rows = min(128, len - mt * 128);
  };

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(TM_REGS_CTRL));
    if (warp == 0) {
      // ---------------------------------------------------------------- TMA producer
      if (lane == 0) {
        const uint64_t pol_w = l2_policy_evict_first();
        const uint64_t pol_x = l2_policy_evict_last();
        uint32_t s = 0, sph = 0;
        uint32_t ag_seen = 0;
        const int ag_round = (p.ag_world > 1) ? *p.ag_epoch : 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
          int g, nt, row0, rows;
          decode_tile(tile, g, nt, row0, rows);
          const int wrow = g * p.w_rows_per_group + (GLU ? nt * TM_BN : nt * 2 * TM_BN);
          const int wrow1 = GLU ? wrow + p.n_out : wrow + TM_BN;
          // activation scales of this tile's rows: [kb][row0 .. row0+128), clipped to the allocation
          const int sc_n = (KIND == 1) ? max(0, min(128, p.x_scale_ld - row0)) : 0;
          if (p.ag_world > 1) {
            // rows of this tile come from ranks s_lo..s_hi; wait until their blocks have landed here
            const int s_lo = row0 / p.ag_rows_per_rank;
            const int s_hi = min(p.ag_world - 1, (row0 + 127) / p.ag_rows_per_rank);
            for (int sr = s_lo; sr <= s_hi && ok; ++sr) {
              if (sr == p.ag_rank || ((ag_seen >> sr) & 1u)) continue;
              if (!flag_wait_ge(p.ag_flag + sr, ag_round, p.ag_wait_ns, p.status, TMS_AG_FLAG, sr)) {
                *abort_flag = 1;
                ok = false;
              }
              ag_seen |= 1u << sr;
            }
            if (!ok) break;
            // the rows were written by peers through the generic proxy; the TMA engine reads through the async one
            asm volatile("fence.proxy.async.global;" ::: "memory");
          }
#pragma unroll 1
          for (int kb = 0; kb < num_kb; ++kb) {
            if (!mbar_wait(&empty_bar[s], sph ^ 1u, abort_flag, p.status, TMS_PROD_EMPTY, (int)s)) { ok = false; break; }
            uint8_t* st = smem + s * L::STAGE_BYTES;
            mbar_expect_tx(&full_bar[s], L::STAGE_BYTES + sc_n * 4);
            tma_load_2d_hint(st, &tmap_x, &full_bar[s], kb * BK_ELEMS + g * p.x_group_col, row0, pol_x);
            tma_load_2d_hint(st + L::A_BYTES, &tmap_w, &full_bar[s], kb * BK_ELEMS, wrow, pol_w);
            tma_load_2d_hint(st + L::A_BYTES + L::B_BYTES, &tmap_w, &full_bar[s], kb * BK_ELEMS, wrow1, pol_w);
            if (sc_n > 0)
              tm_bulk_load_1d(sc_ring + s * 128, p.x_scale + (size_t)kb * p.x_scale_ld + row0, sc_n * 4, &full_bar[s]);
            if (++s == STAGES) { s = 0; sph ^= 1u; }
          }
        }
      }
    } else if (warp == 1) {
      // ---------------------------------------------------------------- MMA issuer (whole warp, one elected lane issues)
      // the two 16 KB weight blocks of a stage are adjacent, which is exactly the K-major layout of 256 rows
      constexpr uint32_t idesc = (KIND == 0) ? umma_idesc(128, 2 * TM_BN, 1, 1) : umma_idesc(128, 2 * TM_BN, 0, 0);
      uint32_t s = 0, sph = 0;
      uint32_t buf = 0, bph = 0;
      bool ok = true;
      const uint32_t smem_base = smem_u32(smem);
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        if (KIND == 0) {   // one accumulator buffer per tile
          if (!mbar_wait(&tempty_bar[buf], bph ^ 1u, abort_flag, p.status, TMS_MMA_TMEM_EMPTY, (int)buf)) { ok = false; break; }
          tc_fence_after();
        }
#pragma unroll 1
        for (int kb = 0; kb < num_kb; ++kb) {
          if (KIND == 1) {
            if (!mbar_wait(&tempty_bar[buf], bph ^ 1u, abort_flag, p.status, TMS_MMA_TMEM_EMPTY, (int)buf)) { ok = false; break; }
          }
          {
            if (!mbar_wait(&full_bar[s], sph, abort_flag, p.status, TMS_MMA_FULL, (int)s)) { ok = false; break; }
          }
          tc_fence_after();
          if (elect_one()) {
            const uint32_t sa = smem_base + s * L::STAGE_BYTES;
            const uint64_t adesc = umma_desc_kmajor_sw128(sa);
            const uint64_t bdesc = umma_desc_kmajor_sw128(sa + L::A_BYTES);
            const uint32_t d0 = tmem_base + buf * ACC_COLS;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              if (KIND == 0) umma_bf16(d0, adesc + 2 * k, bdesc + 2 * k, idesc, (kb != 0 || k != 0) ? 1u : 0u);
              else umma_fp8(d0, adesc + 2 * k, bdesc + 2 * k, idesc, k != 0);
            }
            if (KIND == 0) {
              umma_commit(&empty_bar[s]);                       // operands consumed once these MMAs retire
              if (kb == num_kb - 1) umma_commit(&tfull_bar[buf]);
            } else {
              umma_commit(&tfull_bar[buf]);
            }
          }
          __syncwarp();
          if (KIND == 1) { if (++buf == NBUF) { buf = 0; bph ^= 1u; } }
          if (++s == STAGES) { s = 0; sph ^= 1u; }
        }
        if (KIND == 0) { if (++buf == NBUF) { buf = 0; bph ^= 1u; } }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(TM_REGS_EPI));
    const int q = warp & 3;                 // TMEM lane quadrant this warp may read
    const int grp = (warp - 4) >> 2;        // column half owned by this warp's group
    const int r = q * 32 + lane;            // accumulator lane = token row inside the tile
    const int c_lo = grp * TM_CW;           // first output column (inside the tile) of this group
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    uint32_t s = 0;
    uint32_t buf = 0, bph = 0;
    int sync_no = 0;
    bool ok = true;
    // rendezvous of the eight epilogue warps; watches the abort flag so that nobody can be stranded
    auto epi_sync = [&]() -> bool {
      __syncwarp();
      if (lane == 0) { __threadfence_block(); atomicAdd(epi_counter, 1); }
      ++sync_no;
      uint32_t spins = 0;
      while (*(volatile int*)epi_counter < 8 * sync_no) {
        if (((++spins) & 0xff) == 0 && *abort_flag) return false;
      }
      __syncwarp();
      return true;
    };
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      int g, nt, row0, rows;
      decode_tile(tile, g, nt, row0, rows);
      const int sb_per_group = (p.w_rows_per_group + 127) / 128;
      const int blk0 = GLU ? nt : 2 * nt;
      const int blk1 = GLU ? nt + p.n_out / 128 : 2 * nt + 1;
      const bool blk1_ok = blk1 < sb_per_group;           // store variant: the last tile may have one block only
      const float* wsc0 = (KIND == 1) ? p.w_scale + ((size_t)g * sb_per_group + blk0) * num_kb : nullptr;
      const float* wsc1 = (KIND == 1) ? p.w_scale + ((size_t)g * sb_per_group + (blk1_ok ? blk1 : blk0)) * num_kb : nullptr;

      float2 acc[NB][TM_CW / 2];
#pragma unroll
      for (int a = 0; a < NB; ++a)
#pragma unroll
        for (int j = 0; j < TM_CW / 2; ++j) acc[a][j] = make_float2(0.f, 0.f);

      if (KIND == 0) {
        // the MMA warp accumulated the whole K range in TMEM: fetch the finished tile
        if (!mbar_wait(&tfull_bar[buf], bph, abort_flag, p.status, TMS_EPI_TMEM_FULL, (int)buf)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int a = 0; a < NB; ++a) {
#pragma unroll
          for (int c0 = 0; c0 < TM_CW; c0 += 16) {
            uint32_t v[16];
            tmem_ld_x16(lane_addr + buf * ACC_COLS + a * TM_BN + c_lo + c0, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[a][c0 / 2 + j] = make_float2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty_bar[buf]);
        if (++buf == NBUF) { buf = 0; bph ^= 1u; }
      }
#pragma unroll 1
      for (int kb = 0; KIND == 1 && kb < num_kb; ++kb) {
        // consecutive weight scales share a cache line, so these loads hit L1 except once every 32 K blocks
        const float sw0 = __ldg(wsc0 + kb);
        const float sw1 = blk1_ok ? __ldg(wsc1 + kb) : 0.f;
        {
          if (!mbar_wait(&tfull_bar[buf], bph, abort_flag, p.status, TMS_EPI_TMEM_FULL, (int)buf)) { ok = false; break; }
        }
        tc_fence_after();
        const float sx = sc_ring[s * 128 + r];
#pragma unroll
        for (int a = 0; a < NB; ++a) {
          uint32_t t[TM_CW];
#pragma unroll
          for (int c0 = 0; c0 < TM_CW; c0 += 16) {
            uint32_t v[16];
            tmem_ld_x16(lane_addr + buf * ACC_COLS + a * TM_BN + c_lo + c0, v);
#pragma unroll
            for (int j = 0; j < 16; ++j) t[c0 + j] = v[j];
          }
          tmem_ld_wait();
          if (a == NB - 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
              mbar_arrive(&tempty_bar[buf]);   // the MMA may overwrite this buffer now
              mbar_arrive(&empty_bar[s]);      // scale slot read, MMAs of the stage retired
            }
          }
          const float m = sx * (a == 0 ? sw0 : sw1);
          const float2 m2 = make_float2(m, m);
#pragma unroll
          for (int j = 0; j < TM_CW / 2; ++j)
            tm_fma2(acc[a][j], make_float2(__uint_as_float(t[2 * j]), __uint_as_float(t[2 * j + 1])), m2);
        }
        if (++buf == NBUF) { buf = 0; bph ^= 1u; }
        if (++s == STAGES) s = 0;
      }
      if (!ok) break;

      // ---- per-tile output: this thread owns token row r and columns [n0, n0 + 64) of the output
      const bool row_ok = r < rows;
      const size_t row = (size_t)(row0 + r);
      if (EPI == 0) {
        const float rs = (p.row_scale && row_ok) ? __ldg(p.row_scale + row) : 1.0f;
        if (row_ok) {
          // where this token row goes: the local output, or (reduce-scatter) the receive slab of the rank that
          // owns the row, at [this rank][row inside the owner's block]
          uint8_t* obase = (uint8_t*)p.out;
          size_t orow = row;
          if (p.rs_world > 1) {
            const int dst = (int)(row / (size_t)p.rs_rows_per_rank);
            obase = (uint8_t*)p.rs_out[dst];
            orow = (size_t)p.rs_rank * p.rs_rows_per_rank + (row - (size_t)dst * p.rs_rows_per_rank);
          }
#pragma unroll
          for (int a = 0; a < NB; ++a) {
            const int nl = (2 * nt + a) * TM_BN + c_lo;   // block a = output features [ (2 nt + a) * 128, +128 )
            if (nl >= p.n_out) continue;
            const size_t ocol = (size_t)nl + (size_t)g * p.out_group_col;
            if (p.out_f32) {
              float* o = (float*)obase + orow * p.out_ld + ocol;
#pragma unroll
              for (int j = 0; j < TM_CW / 2; j += 2) {
                if (nl + 2 * j + 3 < p.n_out) {
                  *reinterpret_cast<float4*>(o + 2 * j) =
                      make_float4(acc[a][j].x * rs, acc[a][j].y * rs, acc[a][j + 1].x * rs, acc[a][j + 1].y * rs);
                } else {
                  const float v4[4] = {acc[a][j].x * rs, acc[a][j].y * rs, acc[a][j + 1].x * rs, acc[a][j + 1].y * rs};
                  for (int e = 0; e < 4; ++e)
                    if (nl + 2 * j + e < p.n_out) o[2 * j + e] = v4[e];
                }
              }
            } else {
              __nv_bfloat16* o = (__nv_bfloat16*)obase + orow * p.out_ld + ocol;
              // 32-byte stores where the row allows it: a lane then writes whole 32-byte sectors (the lanes of a
              // warp write 32 different rows, so 16-byte stores would leave every sector half written per instruction)
              const bool wide = (((uintptr_t)o & 31) == 0) && (nl + TM_CW <= p.n_out);
#pragma unroll
              for (int j = 0; j < TM_CW / 2; j += 8) {
                __nv_bfloat162 h[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) h[e] = __floats2bfloat162_rn(acc[a][j + e].x * rs, acc[a][j + e].y * rs);
                if (wide) {
                  const uint32_t* hw = reinterpret_cast<const uint32_t*>(h);
                  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                               ::"l"(o + 2 * j), "r"(hw[0]), "r"(hw[1]), "r"(hw[2]), "r"(hw[3]), "r"(hw[4]), "r"(hw[5]),
                                 "r"(hw[6]), "r"(hw[7])
                               : "memory");
                } else {
#pragma unroll
                  for (int q4 = 0; q4 < 2; ++q4) {
                    if (nl + 2 * j + 8 * q4 + 7 < p.n_out) {
                      *reinterpret_cast<uint4*>(o + 2 * j + 8 * q4) = *reinterpret_cast<uint4*>(h + 4 * q4);
                    } else {
                      const __nv_bfloat16* hv = reinterpret_cast<const __nv_bfloat16*>(h + 4 * q4);
                      for (int e = 0; e < 8; ++e)
                        if (nl + 2 * j + 8 * q4 + e < p.n_out) o[2 * j + 8 * q4 + e] = hv[e];
                    }
                  }
                }
              }
            }
          }
        }
      } else {
        // SwiGLU on (gate, up) held by the same thread; overwrite the gate accumulator with the activation
        const int n0 = nt * TM_BN + c_lo;
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < TM_CW / 2; ++j) {
          acc[0][j].x = silu_f(acc[0][j].x) * acc[NB - 1][j].x;
          acc[0][j].y = silu_f(acc[0][j].y) * acc[NB - 1][j].y;
          amax = fmaxf(amax, fmaxf(fabsf(acc[0][j].x), fabsf(acc[0][j].y)));
        }
        if (EPI == 1) {
          if (row_ok) {
            __nv_bfloat16* o = (__nv_bfloat16*)p.out + row * p.out_ld + n0;
            const bool wide = ((uintptr_t)o & 31) == 0;
#pragma unroll
            for (int j = 0; j < TM_CW / 2; j += 8) {
              __nv_bfloat162 h[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) h[e] = __floats2bfloat162_rn(acc[0][j + e].x, acc[0][j + e].y);
              const uint32_t* hw = reinterpret_cast<const uint32_t*>(h);
              if (wide) {
                asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                             ::"l"(o + 2 * j), "r"(hw[0]), "r"(hw[1]), "r"(hw[2]), "r"(hw[3]), "r"(hw[4]), "r"(hw[5]),
                               "r"(hw[6]), "r"(hw[7])
                             : "memory");
              } else {
                *reinterpret_cast<uint4*>(o + 2 * j) = *reinterpret_cast<const uint4*>(h);
                *reinterpret_cast<uint4*>(o + 2 * j + 8) = *reinterpret_cast<const uint4*>(h + 4);
              }
            }
          }
        } else {
          // the quantisation block is the tile's 128 features: the two threads that share a token row (one in
          // each group) exchange their maxima.  Two rendezvous per tile: after the writes, and after the reads
          // (so that the next tile's writes cannot overtake them).
          amax_x[grp * 128 + r] = amax;
          if (!epi_sync()) { ok = false; break; }
          const float mx = fmaxf(amax_x[r], amax_x[128 + r]);
          if (!epi_sync()) { ok = false; break; }
          const float scl = fmaxf(mx, 1e-10f) * (1.0f / 448.0f);
          const float inv = 1.0f / scl;
          if (row_ok) {
            uint8_t* o = (uint8_t*)p.out + row * p.out_ld + n0;
            const bool wide = ((uintptr_t)o & 31) == 0;
#pragma unroll
            for (int j = 0; j < TM_CW / 2; j += 16) {
              __align__(16) uint8_t b[32];
#pragma unroll
              for (int e = 0; e < 16; ++e) {
                b[2 * e] = f32_to_e4m3(acc[0][j + e].x * inv);
                b[2 * e + 1] = f32_to_e4m3(acc[0][j + e].y * inv);
              }
              const uint32_t* bw = reinterpret_cast<const uint32_t*>(b);
              if (wide) {
                asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                             ::"l"(o + 2 * j), "r"(bw[0]), "r"(bw[1]), "r"(bw[2]), "r"(bw[3]), "r"(bw[4]), "r"(bw[5]),
                               "r"(bw[6]), "r"(bw[7])
                             : "memory");
              } else {
                *reinterpret_cast<uint4*>(o + 2 * j) = *reinterpret_cast<const uint4*>(b);
                *reinterpret_cast<uint4*>(o + 2 * j + 16) = *reinterpret_cast<const uint4*>(b + 16);
              }
            }
            if (grp == 0) p.out_scale[(size_t)nt * p.out_scale_ld + row] = scl;
          }
        }
      }
    }
  }

  // ------------------------------------------------------------------ reduce-scatter: tell the destinations
  if (p.rs_world > 1) {
    if (warp >= 4) __threadfence_system();   // this thread's peer stores are performed before the flag below
    __syncthreads();
    if (threadIdx.x == 0 && !*abort_flag) {
      __threadfence();
      const int done = atomicAdd(p.rs_done, 1);
      if (done == (int)gridDim.x - 1) {      // every CTA of this rank has written its rows
        *p.rs_done = 0;                       // ready for the next launch
        const int round = *p.rs_epoch + 1;    // kept in device memory so that a replayed CUDA graph advances it too
        *p.rs_epoch = round;
        __threadfence_system();
        for (int d = 0; d < p.rs_world; ++d) st_release_sys(p.rs_flag[d], round);
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  if (*abort_flag) {
    if (threadIdx.x == 0) report_abort(abort_flag, p.status);
    // give copies that are still in flight time to land before the CTA's memory is released
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int KIND, int EPI>
static int launch_tm(const CUtensorMap& tx, const CUtensorMap& tw, const TmGemmParams& p, int grid, cudaStream_t st) {
  using L = TmSmem;
  auto kfn = gemm_tokmajor_kernel<KIND, EPI>;
  static bool configured[64] = {false};
  if (int e = ensure_dyn_smem((const void*)kfn, L::TOTAL, configured)) return e;
  kfn<<<grid, TM_THREADS, L::TOTAL, st>>>(tx, tw, p);
  return (int)cudaGetLastError();
}

}  // namespace omni

using namespace omni;


// Collective side of a call (all zero / null for a plain GEMM).
struct OmniTmCollective {
  int rs_world, rs_rank, rs_rows_per_rank, pad0;
  void* rs_out[8];
  int* rs_flag[8];
  int* rs_done;
  int* rs_epoch;
  int ag_world, ag_rank, ag_rows_per_rank, pad1;
  const int* ag_flag;
  const int* ag_epoch;
  unsigned long long ag_wait_ns;
};

// Token-major GEMM.  kind: 0 bf16, 1 e4m3 block-scaled.  Arguments as omni_gemm; `coll` may be null.
// Requirements beyond omni_gemm's: n_out a multiple of 8 (16-byte output vectors), for the SwiGLU variants a
// multiple of 128; segment starts a multiple of 4 rows for e4m3 (bulk copies of activation scales); out_ld a
// multiple of 8 elements.  Returns 0 on success, a negative value for bad arguments, a positive CUDA error
// otherwise.
extern "C" int omni_gemm_tm2(int kind, int epi, const void* w, const void* x, void* out, int G, int n_out, int K, int x_rows,
                             int T, const int* seg_start, const int* seg_len, const float* w_scale, const float* x_scale,
                             int x_scale_ld, int out_ld, int out_f32, float* out_scale, int out_scale_ld,
                             const float* row_scale, int x_group_col, int out_group_col, int x_ld,
                             const OmniTmCollective* coll, void* status, cudaStream_t stream) {
  if (G < 1 || G > TM_MAX_GROUPS || n_out < 1 || K < 1) return -1;
  if (kind != 0 && kind != 1) return -1;
  const int nb = (epi == 0) ? 1 : 2;
  const int esz = (kind == 0) ? 2 : 1;
  if ((K * esz) % 16 != 0) return -2;
  if (nb == 2 && (n_out % 128) != 0) return -3;
  if (kind == 1 && (w_scale == nullptr || x_scale == nullptr)) return -4;
  if (kind == 1 && ((x_scale_ld % 4) != 0 || ((uintptr_t)x_scale % 16) != 0)) return -7;
  if (epi == 2 && (out_scale == nullptr || kind != 1)) return -5;
  if ((n_out % 8) != 0 || (out_ld % 8) != 0 || (out_group_col % 8) != 0) return -8;
  if (epi < 0 || epi > 2) return -9;
  TmGemmParams p;
  memset(&p, 0, sizeof(p));
  p.G = G; p.n_out = n_out; p.K = K; p.T = T; p.seg_start = seg_start; p.seg_len = seg_len;
  p.w_rows_per_group = n_out * nb; p.w_scale = w_scale; p.x_scale = x_scale; p.x_scale_ld = x_scale_ld;
  p.out = out; p.out_ld = out_ld; p.out_f32 = out_f32; p.out_scale = out_scale; p.out_scale_ld = out_scale_ld;
  p.row_scale = row_scale; p.x_group_col = x_group_col; p.out_group_col = out_group_col; p.status = (OmniStatus*)status;
  p.rs_world = 1; p.ag_world = 1;
  if (coll != nullptr) {
    if (coll->rs_world > 1) {
      if (coll->rs_world > 8 || epi != 0 || out_f32 || G != 1 || seg_len != nullptr || coll->rs_rows_per_rank < 1) return -12;
      p.rs_world = coll->rs_world; p.rs_rank = coll->rs_rank; p.rs_rows_per_rank = coll->rs_rows_per_rank;
      p.rs_epoch = coll->rs_epoch; p.rs_done = coll->rs_done;
      if (p.rs_epoch == nullptr) return -12;
      for (int d = 0; d < coll->rs_world; ++d) {
        if (coll->rs_out[d] == nullptr || coll->rs_flag[d] == nullptr || ((uintptr_t)coll->rs_out[d] % 16) != 0) return -12;
        p.rs_out[d] = coll->rs_out[d]; p.rs_flag[d] = coll->rs_flag[d];
      }
      if (p.rs_done == nullptr || (long long)coll->rs_world * coll->rs_rows_per_rank < T) return -12;
    }
    if (coll->ag_world > 1) {
      if (coll->ag_world > 8 || G != 1 || seg_len != nullptr || coll->ag_flag == nullptr || coll->ag_rows_per_rank < 1) return -13;
      p.ag_world = coll->ag_world; p.ag_rank = coll->ag_rank; p.ag_rows_per_rank = coll->ag_rows_per_rank;
      p.ag_epoch = coll->ag_epoch; p.ag_flag = coll->ag_flag; p.ag_wait_ns = coll->ag_wait_ns;
      if (p.ag_epoch == nullptr) return -13;
    }
  }
  if (p.rs_world == 1 && ((uintptr_t)out % 16) != 0) return -8;
  if (x_ld <= 0) x_ld = K;
  const uint64_t x_cols = x_group_col > 0 ? (uint64_t)x_ld : (uint64_t)K;
  const int bk = (kind == 0) ? 64 : 128;
  if (x_group_col > 0 && (K % bk) != 0) return -6;   // a K tail would read the next group's columns
  CUtensorMap tx, tw;
  if (make_tmap_2d(&tx, x, esz, (uint64_t)x_rows, x_cols, x_ld, 128, bk, true)) return -11;
  if (make_tmap_2d(&tw, w, esz, (uint64_t)G * p.w_rows_per_group, K, K, TM_BN, bk, true)) return -10;
  const int grid = sm_count();
  if (kind == 0) {
    if (epi == 0) return launch_tm<0, 0>(tx, tw, p, grid, stream);
    if (epi == 1) return launch_tm<0, 1>(tx, tw, p, grid, stream);
    return -9;
  }
  if (epi == 0) return launch_tm<1, 0>(tx, tw, p, grid, stream);
  if (epi == 1) return launch_tm<1, 1>(tx, tw, p, grid, stream);
  return launch_tm<1, 2>(tx, tw, p, grid, stream);
}
