// Weight-stationary ("swap-AB") tcgen05 GEMM family for sm_100a.
//
//   out[t, n] = sum_k X[t, k] * W[g, n, k]            (t in group g's row segment)
//
// The weight rows are the UMMA M dimension (always 128 per tile), the token rows are the UMMA N
// dimension (BN = 16..256), so a decode step with a few dozen tokens per expert still issues
// full-width tensor-core instructions and each weight byte is streamed from HBM exactly once.
// Both operands are K-major in global memory ([rows, K] row-major), staged by TMA into
// 128-byte-swizzled shared memory, multiplied by tcgen05.mma with fp32 accumulators in TMEM.
//
// One persistent CTA per SM, three roles:
//   warp 0      TMA producer (one lane)
//   warp 1      TMEM allocation + MMA issue (one lane)
//   warps 2..9  epilogue (two groups of four, each group owns half of the token columns): tcgen05.ld of the
//               accumulator lanes, scaling, activation, stores
//
// Variants (template parameters):
//   KIND  0 = bf16 operands (accumulate the whole K range in TMEM).  This is the kernel's main use: the fp8
//             GEMMs of the models run on the token-major kernel in gemm_tokmajor_sm100.cu, which promotes
//             with one multiplier per thread; the fp8 kind here is kept as the alternative orientation.
//         1 = e4m3 operands with DeepSeek-style block scales: W scale per 128x128 block, X scale
//             per (row, 128-wide K block).  Every 128-wide K block is multiplied into a fresh
//             TMEM buffer (two buffers ping-pong) and promoted into fp32 registers with
//             w_scale * x_scale by the epilogue warps.
//   NACC  1 = one accumulator; 2 = two weight tiles (gate rows, up rows) share the X tile
//   EPI   0 = store (optional per-row multiplier, bf16 or fp32 output)
//         1 = SwiGLU: silu(gate) * up -> bf16
//         2 = SwiGLU then e4m3 quantisation with one scale per (row, 128 output features);
//             the 128 accumulator lanes of a tile are exactly one quantisation block.
//
// Covers what the reference gets from its vendor ops npu_quant_matmul, npu_grouped_matmul,
// npu_dequant_swiglu_quant and npu_swiglu
// (omni/models/common/layers/moe/fused_moe/fused_moe.py:541-575,
//  omni/quantization/compressed_tensors/compressed_tensors_moe.py:221-253,
//  omni/quantization/compressed_tensors/schemes/compressed_tensors_w8a8_int8.py:84-109).
#include "../include/omni_ptx.cuh"
#include "../include/tma_host.h"

namespace omni {

struct GemmParams {
  int G;                 // groups (experts); 1 for a dense GEMM
  int n_out;             // output features per group and accumulator
  int K;
  int T;                 // rows when seg_* are null
  const int* seg_start;  // [G] first row of the group's segment in X/out, or null
  const int* seg_len;    // [G] rows in the segment, or null
  int w_rows_per_group;  // rows of one group in the flattened weight matrix (n_out * NACC)
  const float* w_scale;  // [G, w_rows_per_group/128, ceil(K/128)]
  const float* x_scale;  // [ceil(K/128), x_scale_ld]
  int x_scale_ld;
  void* out;
  int out_ld;
  int out_f32;
  float* out_scale;      // EPI 2: [n_out/128, out_scale_ld]
  int out_scale_ld;
  const float* row_scale;  // optional [rows]
  int x_group_col;       // head-batched mode: group g reads X columns [g*x_group_col, +K) ...
  int out_group_col;     // ... and writes out columns [g*out_group_col, +n_out)
  int k_splits;          // > 1: the K range is cut into k_splits parts that different CTAs accumulate into a
  int kb_per_split;      //      zero-initialised fp32 output with atomic adds (EPI 0 only); K blocks per part
  OmniStatus* status;
};

constexpr int GEMM_THREADS = 320;     // warp 0 TMA, warp 1 MMA, warps 2..9 epilogue (two groups of four)
constexpr int MAX_GROUPS = 1024;
constexpr int SMEM_BUDGET = 225 * 1024;
constexpr int MAX_STAGES = 10;

template <int BN, int NACC>
struct GemmSmem {
  static constexpr int A_BYTES = 128 * 128;          // 128 weight rows x 128 B
  static constexpr int B_BYTES = BN * 128;
  static constexpr int STAGE_BYTES = NACC * A_BYTES + B_BYTES;
  static constexpr int SC_BYTES = MAX_STAGES * BN * 4;   // activation-scale ring (fp8 kind)
  static constexpr int PREFIX_BYTES = (MAX_GROUPS + 4) * 4;   // G+1 ints, padded so what follows stays 16-byte aligned
  static constexpr int AUX_BYTES = 1024 /*barriers*/ + PREFIX_BYTES + 1024 /*amax exchange*/ + SC_BYTES;
  static constexpr int STAGES_RAW = (SMEM_BUDGET - AUX_BYTES - 1024) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > MAX_STAGES ? MAX_STAGES : STAGES_RAW;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + AUX_BYTES + 1024;
};

enum { SITE_PROD_EMPTY = 1, SITE_MMA_FULL = 2, SITE_MMA_TMEM_EMPTY = 3, SITE_EPI_TMEM_FULL = 4, SITE_TMEM_BASE = 5 };

__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// packed fp32 pair arithmetic (two lanes per instruction)
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
  float2 d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(reinterpret_cast<uint64_t&>(d))
      : "l"(reinterpret_cast<uint64_t&>(a)), "l"(reinterpret_cast<uint64_t&>(b)));
  return d;
}
__device__ __forceinline__ void fma2(float2& acc, float2 a, float2 b) {
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(reinterpret_cast<uint64_t&>(acc))
      : "l"(reinterpret_cast<uint64_t&>(a)), "l"(reinterpret_cast<uint64_t&>(b)));
}

#define GT_BEGIN
#define GT_END(slot)

template <int KIND, int BN, int NACC, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_swapab_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                   const GemmParams p) {
  using L = GemmSmem<BN, NACC>;
  constexpr int STAGES = L::STAGES;
  constexpr int BK_ELEMS = (KIND == 0) ? 64 : 128;       // one 128-byte swizzle span
  constexpr int ACC_COLS = NACC * BN;                    // TMEM columns of one accumulator buffer
  constexpr int CW = BN / 2;                             // token columns owned by one epilogue group
  // One CTA per SM, so it takes the whole TMEM: the allocation then starts at column 0 and every TMEM address
  // is a compile-time constant.  (tcgen05.mma issues several times slower when its operands have to be moved
  // over from ordinary registers, as a base address loaded from shared memory would be.)
  constexpr int TMEM_COLS = 512;
  static_assert(2 * ACC_COLS <= 512, "accumulators exceed TMEM");
  static_assert(BN % 32 == 0 && BN >= 32 && BN <= 256, "invalid token tile");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* aux = smem + STAGES * L::STAGE_BYTES;
  uint64_t* full_bar = (uint64_t*)aux;                   // [STAGES]
  uint64_t* empty_bar = full_bar + MAX_STAGES;           // [STAGES]
  uint64_t* tfull_bar = empty_bar + MAX_STAGES;          // [2]
  uint64_t* tempty_bar = tfull_bar + 2;                  // [2]
  uint32_t* tmem_slot = (uint32_t*)(tempty_bar + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  int* epi_counter = (int*)(tmem_slot + 2);              // [2] one per epilogue group
  int* tile_prefix = (int*)(aux + 1024);                 // [G + 1]
  float* amax_x = (float*)(aux + 1024 + L::PREFIX_BYTES);  // [2 groups][2 slabs][4 warps][16]
  float* sc_ring = amax_x + 256;                         // [STAGES][BN], 16-byte aligned (bulk copies, float4 reads)
  static_assert((1024 + L::PREFIX_BYTES + 1024) % 16 == 0, "scale ring must be 16-byte aligned");

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb = (p.K + BK_ELEMS - 1) / BK_ELEMS;
  const int m_tiles = (p.n_out + 127) / 128;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      // bf16: released by the MMA commit.  fp8: released by the 8 epilogue warps once they have read the stage's
      // scale-ring slot, which they only do after the stage's MMAs have retired (they waited for tfull).
      mbar_init(&empty_bar[s], (KIND == 1) ? 8 : 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull_bar[b], 1);
      mbar_init(&tempty_bar[b], 8);
    }
    *abort_flag = 0;
    epi_counter[0] = 0;
    epi_counter[1] = 0;
    mbar_fence_init();
    // tiles per group: ceil(len / BN) * m_tiles, token tile fastest
    int acc = 0;
    for (int g = 0; g < p.G; ++g) {
      tile_prefix[g] = acc;
      int len = p.seg_len ? p.seg_len[g] : p.T;
      acc += ((len + BN - 1) / BN) * m_tiles;
    }
    tile_prefix[p.G] = acc;
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  constexpr uint32_t tmem_base = 0;
  if (*tmem_slot != 0u) {   // cannot happen while the whole TMEM is requested; never compute on a wrong base
    if (threadIdx.x == 0) { *abort_flag = 1; report_status(p.status, OMNI_ERR_MBAR_TIMEOUT, SITE_TMEM_BASE, (int)*tmem_slot); }
    __syncthreads();
    if (warp == 1) tmem_dealloc(*tmem_slot, TMEM_COLS);
    return;
  }
  const int total_tiles = tile_prefix[p.G];

  // tile index -> (group, m_tile, n_tile, first row, rows valid)
  auto decode_tile = [&](int tile, int& g, int& mt, int& row0, int& rows) {
    int lo = 0, hi = p.G - 1;
    while (lo < hi) {  // last g with tile_prefix[g] <= tile
      int mid = (lo + hi + 1) >> 1;
      if (tile_prefix[mid] <= tile) lo = mid; else hi = mid - 1;
    }
    g = lo;
    int local = tile - tile_prefix[g];
    int len = p.seg_len ? p.seg_len[g] : p.T;
    int n_tiles = (len + BN - 1) / BN;
    mt = local / n_tiles;
    int nt = local - mt * n_tiles;
    int start = p.seg_start ? p.seg_start[g] : 0;
    row0 = start + nt * BN;
    rows = min(BN, len - nt * BN);
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const uint64_t pol_w = l2_policy_evict_first();
      const uint64_t pol_x = l2_policy_evict_last();
      uint32_t s = 0, sph = 0;
      bool ok = true;
      for (int vt = blockIdx.x; vt < total_tiles * p.k_splits && ok; vt += gridDim.x) {
        const int tile = vt / p.k_splits;
        const int kb0 = (vt - tile * p.k_splits) * p.kb_per_split;
        const int kb1 = min(num_kb, kb0 + p.kb_per_split);
        int g, mt, row0, rows;
        decode_tile(tile, g, mt, row0, rows);
        const int wrow = g * p.w_rows_per_group + mt * 128;
        // activation scales of this tile's rows: [kb][row0 .. row0+BN), clipped to the allocation
        const int sc_n = (KIND == 1) ? max(0, min(BN, p.x_scale_ld - row0)) : 0;
#pragma unroll 1
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[s], sph ^ 1u, abort_flag, p.status, SITE_PROD_EMPTY, (int)s)) { ok = false; break; }
          uint8_t* st = smem + s * L::STAGE_BYTES;
          mbar_expect_tx(&full_bar[s], L::STAGE_BYTES + sc_n * 4);
          tma_load_2d_hint(st, &tmap_w, &full_bar[s], kb * BK_ELEMS, wrow, pol_w);
          if (NACC == 2)
            tma_load_2d_hint(st + L::A_BYTES, &tmap_w, &full_bar[s], kb * BK_ELEMS, wrow + p.n_out, pol_w);
          tma_load_2d_hint(st + NACC * L::A_BYTES, &tmap_x, &full_bar[s], kb * BK_ELEMS + g * p.x_group_col, row0, pol_x);
          if (KIND == 1 && sc_n > 0)
            bulk_load_1d(sc_ring + s * BN, p.x_scale + (size_t)kb * p.x_scale_ld + row0, sc_n * 4, &full_bar[s]);
          if (++s == STAGES) { s = 0; sph ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // The whole warp runs the (small) loop and waits on the barriers; one elected lane issues.  That keeps the
    // warp convergent, which measurably shortens the issue path of tcgen05.mma.
    {
      constexpr uint32_t idesc = (KIND == 0) ? umma_idesc(128, BN, 1, 1) : umma_idesc(128, BN, 0, 0);
      uint32_t s = 0, sph = 0;   // smem stage and its phase
      int acc_it = 0;            // accumulator buffer counter
      bool ok = true;
      const uint32_t smem_base = smem_u32(smem);
      for (int vt = blockIdx.x; vt < total_tiles * p.k_splits && ok; vt += gridDim.x) {
        const int tile = vt / p.k_splits;
        const int kb0 = (vt - tile * p.k_splits) * p.kb_per_split;
        const int kb1 = min(num_kb, kb0 + p.kb_per_split);
        if (KIND == 0) {
          const int buf = acc_it & 1;
          if (!mbar_wait(&tempty_bar[buf], ((acc_it >> 1) & 1) ^ 1, abort_flag, p.status, SITE_MMA_TMEM_EMPTY, buf)) {
            ok = false; break;
          }
          tc_fence_after();
        }
#pragma unroll 1
        for (int kb = kb0; kb < kb1; ++kb) {
          const int buf = acc_it & 1;
          if (KIND == 1) {
            GT_BEGIN;
            if (!mbar_wait(&tempty_bar[buf], ((acc_it >> 1) & 1) ^ 1, abort_flag, p.status, SITE_MMA_TMEM_EMPTY, buf)) {
              ok = false; break;
            }
            GT_END(0);
          }
          {
            GT_BEGIN;
            if (!mbar_wait(&full_bar[s], sph, abort_flag, p.status, SITE_MMA_FULL, (int)s)) { ok = false; break; }
            GT_END(1);
          }
          tc_fence_after();
          if (elect_one()) {
            const uint32_t sa = smem_base + s * L::STAGE_BYTES;
            const uint64_t adesc = umma_desc_kmajor_sw128(sa);
            const uint64_t adesc2 = umma_desc_kmajor_sw128(sa + L::A_BYTES);
            const uint64_t bdesc = umma_desc_kmajor_sw128(sa + NACC * L::A_BYTES);
            const uint32_t d0 = tmem_base + buf * ACC_COLS;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const uint32_t accum = (KIND == 0) ? (kb != kb0 || k != 0) : (k != 0);
              if (KIND == 0) {
                umma_bf16(d0, adesc + 2 * k, bdesc + 2 * k, idesc, accum);
                if (NACC == 2) umma_bf16(d0 + BN, adesc2 + 2 * k, bdesc + 2 * k, idesc, accum);
              } else {
                umma_fp8(d0, adesc + 2 * k, bdesc + 2 * k, idesc, accum);
                if (NACC == 2) umma_fp8(d0 + BN, adesc2 + 2 * k, bdesc + 2 * k, idesc, accum);
              }
            }
            if (KIND == 0) umma_commit(&empty_bar[s]);  // operands consumed once these MMAs retire
            else umma_commit(&tfull_bar[buf]);
          }
          __syncwarp();
          if (KIND == 1) ++acc_it;
          if (++s == STAGES) { s = 0; sph ^= 1u; }
        }
        if (KIND == 0 && ok) {
          if (elect_one()) umma_commit(&tfull_bar[acc_it & 1]);
          __syncwarp();
          ++acc_it;
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps
    const int q = warp & 3;                 // TMEM lane quadrant this warp may read
    const int grp = (warp - 2) >> 2;        // column half owned by this warp's group
    const int r = q * 32 + lane;            // accumulator lane = weight row inside the tile
    const int c_lo = grp * CW;              // first token column of this group
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    int acc_it = 0;
    uint32_t s = 0;                         // smem stage whose scale-ring slot belongs to the current K block
    int epi_sync = 0;
    bool ok = true;
    for (int vt = blockIdx.x; vt < total_tiles * p.k_splits && ok; vt += gridDim.x) {
        const int tile = vt / p.k_splits;
        const int kb0 = (vt - tile * p.k_splits) * p.kb_per_split;
        const int kb1 = min(num_kb, kb0 + p.kb_per_split);
      int g, mt, row0, rows;
      decode_tile(tile, g, mt, row0, rows);
      const int n_in = mt * 128 + r;
      const bool n_ok = n_in < p.n_out;
      const int n = n_in + g * p.out_group_col;  // output column

      float2 acc[(KIND == 1) ? NACC * CW / 2 : 1];
      if (KIND == 1) {
#pragma unroll
        for (int j = 0; j < NACC * CW / 2; ++j) acc[j] = make_float2(0.f, 0.f);
        const int sb_per_group = p.w_rows_per_group / 128;
        const float* wsc0 = p.w_scale + ((size_t)g * sb_per_group + mt) * num_kb;
        const float* wsc1 = p.w_scale + ((size_t)g * sb_per_group + mt + p.n_out / 128) * num_kb;
#pragma unroll 1
        for (int kb = kb0; kb < kb1; ++kb, ++acc_it) {
          const int buf = acc_it & 1;
          {
            GT_BEGIN;
            if (!mbar_wait(&tfull_bar[buf], (acc_it >> 1) & 1, abort_flag, p.status, SITE_EPI_TMEM_FULL, buf)) {
              ok = false; break;
            }
            GT_END(2);
          }
          tc_fence_after();
          // pull this group's columns of the fresh partial product out of TMEM in one round trip
          uint32_t t[NACC][CW];
#pragma unroll
          for (int a = 0; a < NACC; ++a) {
#pragma unroll
            for (int c0 = 0; c0 < CW; c0 += 16) {
              uint32_t v[16];
              tmem_ld_x16(lane_addr + buf * ACC_COLS + a * BN + c_lo + c0, v);
#pragma unroll
              for (int j = 0; j < 16; ++j) t[a][c0 + j] = v[j];
            }
          }
          const float sw0 = __ldg(wsc0 + kb);
          const float sw1 = (NACC == 2) ? __ldg(wsc1 + kb) : 0.f;
          tmem_ld_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tempty_bar[buf]);   // the MMA may overwrite this buffer now
          // acc += t * (x_scale * w_scale), sixteen columns at a time.  The scale reads of the next chunk are
          // issued before the arithmetic of this one and the products are formed in a batch, so that neither the
          // shared-memory latency nor the multiply -> fma dependency sits between consecutive instructions.
          const float4* sc4 = reinterpret_cast<const float4*>(sc_ring + s * BN + c_lo);
          const float2 w0 = make_float2(sw0, sw0), w1 = make_float2(sw1, sw1);
          constexpr int NCH = CW / 16;
          float4 sxc[4];
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) sxc[q4] = sc4[q4];
#pragma unroll
          for (int c = 0; c < NCH; ++c) {
            float4 nxt[4];
            if (c + 1 < NCH) {
#pragma unroll
              for (int q4 = 0; q4 < 4; ++q4) nxt[q4] = sc4[(c + 1) * 4 + q4];
            }
            float2 pr[NACC][8];
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
#pragma unroll
              for (int a = 0; a < NACC; ++a) {
                const float2 wa = (a == 0) ? w0 : w1;
                pr[a][2 * q4] = mul2(make_float2(sxc[q4].x, sxc[q4].y), wa);
                pr[a][2 * q4 + 1] = mul2(make_float2(sxc[q4].z, sxc[q4].w), wa);
              }
            }
#pragma unroll
            for (int h = 0; h < 8; ++h) {
#pragma unroll
              for (int a = 0; a < NACC; ++a) {
                const int col = c * 16 + 2 * h;
                fma2(acc[a * CW / 2 + col / 2], make_float2(__uint_as_float(t[a][col]), __uint_as_float(t[a][col + 1])), pr[a][h]);
              }
            }
            if (c + 1 < NCH) {
#pragma unroll
              for (int q4 = 0; q4 < 4; ++q4) sxc[q4] = nxt[q4];
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&empty_bar[s]);      // scale ring slot read
          if (++s == STAGES) s = 0;
        }
        if (!ok) break;
      } else {
        const int buf = acc_it & 1;
        if (!mbar_wait(&tfull_bar[buf], (acc_it >> 1) & 1, abort_flag, p.status, SITE_EPI_TMEM_FULL, buf)) {
          ok = false; break;
        }
        tc_fence_after();
      }

      // ---- per-tile output: this thread owns weight row r and token columns [c_lo, c_lo + CW)
      const int bufc = acc_it & 1;  // bf16 path: buffer holding this tile
      auto accv = [&](int a, int j) -> float {   // fp8 path: accumulator a, local column j
        const float2 v = acc[(KIND == 1) ? (a * CW / 2 + (j >> 1)) : 0];
        return (j & 1) ? v.y : v.x;
      };
      if (EPI == 0) {
#pragma unroll
        for (int c0 = 0; c0 < CW; c0 += 16) {
          float vals[16];
          if (KIND == 0) {
            uint32_t v[16];
            tmem_ld_x16(lane_addr + bufc * ACC_COLS + c_lo + c0, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) vals[j] = __uint_as_float(v[j]);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) vals[j] = accv(0, c0 + j);
          }
          if (c_lo + c0 < rows && n_ok) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              if (c_lo + c0 + j < rows) {
                const size_t row = (size_t)(row0 + c_lo + c0 + j);
                float y = vals[j];
                if (p.row_scale) y *= __ldg(p.row_scale + row);
                if (p.k_splits > 1) atomicAdd((float*)p.out + row * p.out_ld + n, y);
                else if (p.out_f32) ((float*)p.out)[row * p.out_ld + n] = y;
                else ((__nv_bfloat16*)p.out)[row * p.out_ld + n] = __float2bfloat16(y);
              }
            }
          }
        }
      } else {
        // SwiGLU on (gate, up) held by the same lane
#pragma unroll
        for (int c0 = 0; c0 < CW; c0 += 16) {
          float act[16];
          if (KIND == 0) {
            uint32_t vg[16], vu[16];
            tmem_ld_x16(lane_addr + bufc * ACC_COLS + c_lo + c0, vg);
            tmem_ld_x16(lane_addr + bufc * ACC_COLS + BN + c_lo + c0, vu);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) act[j] = silu_f(__uint_as_float(vg[j])) * __uint_as_float(vu[j]);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) act[j] = silu_f(accv(0, c0 + j)) * accv(NACC - 1, c0 + j);
          }
          if (EPI == 1) {
            if (c_lo + c0 < rows && n_ok) {
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (c_lo + c0 + j < rows)
                  ((__nv_bfloat16*)p.out)[(size_t)(row0 + c_lo + c0 + j) * p.out_ld + n] = __float2bfloat16(act[j]);
            }
          } else {
            // amax over the 128 lanes of the tile for each of the 16 token columns.  The four warps of
            // this group exchange their partial maxima through a double-buffered slab and a counter
            // that only grows; the wait on the counter also watches the abort flag, so a warp
            // that left early can never strand the others (a bar.sync could).
            float* slab = amax_x + grp * 128 + (epi_sync & 1) * 64;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              float m = warp_max(n_ok ? fabsf(act[j]) : 0.f);
              if (lane == 0) slab[q * 16 + j] = m;
            }
            __syncwarp();
            if (lane == 0) {
              __threadfence_block();
              atomicAdd(&epi_counter[grp], 1);
            }
            ++epi_sync;
            {
              uint32_t spins = 0;
              while (*(volatile int*)&epi_counter[grp] < 4 * epi_sync) {
                if (((++spins) & 0xff) == 0 && *abort_flag) { ok = false; break; }
              }
              __syncwarp();
              if (!ok) break;
            }
            float scl[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              float m = fmaxf(fmaxf(slab[j], slab[16 + j]), fmaxf(slab[32 + j], slab[48 + j]));
              scl[j] = fmaxf(m, 1e-10f) * (1.0f / 448.0f);
            }
            if (c_lo + c0 < rows) {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                if (c_lo + c0 + j < rows) {
                  const size_t row = (size_t)(row0 + c_lo + c0 + j);
                  if (n_ok) ((uint8_t*)p.out)[row * p.out_ld + n] = f32_to_e4m3(act[j] / scl[j]);
                  if (r == 0) p.out_scale[(size_t)mt * p.out_scale_ld + row] = scl[j];
                }
              }
            }
          }
        }
      }
      if (KIND == 0) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty_bar[bufc]);
        ++acc_it;
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
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// -------------------------------------------------------------------------------------------
// host side
// -------------------------------------------------------------------------------------------
template <int KIND, int BN, int NACC, int EPI>
static int launch_gemm(const CUtensorMap& tw, const CUtensorMap& tx, const GemmParams& p, int grid, cudaStream_t st) {
  using L = GemmSmem<BN, NACC>;
  auto kfn = gemm_swapab_kernel<KIND, BN, NACC, EPI>;
  static bool configured[64] = {false};
  if (int e = ensure_dyn_smem((const void*)kfn, L::TOTAL, configured)) return e;
  kfn<<<grid, GEMM_THREADS, L::TOTAL, st>>>(tw, tx, p);
  return (int)cudaGetLastError();
}

}  // namespace omni

using namespace omni;


// kind: 0 bf16, 1 fp8 block-scaled.  epi: 0 store, 1 swiglu->bf16, 2 swiglu->fp8+scales.
// bn: token tile (16, 32, 64, 128, 256); 0 picks from `t_hint` (expected rows per group).
// x_rows: number of addressable rows of X (and of `out`); rows beyond it read as zero.
// Returns 0 on success, a negative value for bad arguments, a positive CUDA error otherwise.
extern "C" int omni_gemm(int kind, int epi, const void* w, const void* x, void* out, int G, int n_out, int K,
                         int x_rows, int T, const int* seg_start, const int* seg_len, const float* w_scale,
                         const float* x_scale, int x_scale_ld, int out_ld, int out_f32, float* out_scale,
                         int out_scale_ld, const float* row_scale, int x_group_col, int out_group_col, int x_ld,
                         int bn, int t_hint, void* status, cudaStream_t stream) {
  if (G < 1 || G > MAX_GROUPS || n_out < 1 || K < 1) return -1;
  const int nacc = (epi == 0) ? 1 : 2;
  const int esz = (kind == 0) ? 2 : 1;
  if ((K * esz) % 16 != 0) return -2;
  if (nacc == 2 && (n_out % 128) != 0) return -3;
  if (kind == 1 && (w_scale == nullptr || x_scale == nullptr)) return -4;
  if (kind == 1 && ((x_scale_ld % 4) != 0 || ((uintptr_t)x_scale % 16) != 0)) return -7;  // bulk copies of scale rows
  if (epi == 2 && out_scale == nullptr) return -5;
  if (bn == 0) {
    int t = t_hint > 0 ? t_hint : T;
    const int cap = (kind == 1) ? (nacc == 2 ? 64 : 128) : (nacc == 2 ? 128 : 256);
    bn = t <= 32 ? 32 : t <= 64 ? 64 : t <= 128 ? 128 : 256;
    if (bn > cap) bn = cap;
  }
  if (bn == 16) bn = 32;   // smallest instantiated token tile
  // Few output tiles and a long K (the router): cut K so that the whole GPU works on it.  Needs an fp32
  // output that this call may zero first (dense rows, no per-row multiplier).
  int k_splits = 1;
  const int num_kb_h = (K + ((kind == 0) ? 64 : 128) - 1) / ((kind == 0) ? 64 : 128);
  if (epi == 0 && out_f32 && G == 1 && seg_len == nullptr && row_scale == nullptr && out_group_col == 0 && out_ld == n_out) {
    if (bn > 128) bn = 128;
    const int tiles = ((n_out + 127) / 128) * ((T + bn - 1) / bn);
    const int sms = sm_count();
    if (tiles * 2 <= sms && num_kb_h >= 8) {
      k_splits = sms / tiles;
      if (k_splits > num_kb_h / 4) k_splits = num_kb_h / 4;
      if (k_splits > 32) k_splits = 32;
      if (k_splits < 1) k_splits = 1;
    }
  }
  GemmParams p;
  p.kb_per_split = (num_kb_h + k_splits - 1) / k_splits;
  k_splits = (num_kb_h + p.kb_per_split - 1) / p.kb_per_split;   // no empty parts
  p.k_splits = k_splits;
  if (k_splits > 1) {
    cudaError_t e = cudaMemsetAsync(out, 0, (size_t)T * out_ld * sizeof(float), stream);
    if (e != cudaSuccess) return (int)e;
  }
  p.G = G; p.n_out = n_out; p.K = K; p.T = T; p.seg_start = seg_start; p.seg_len = seg_len;
  p.w_rows_per_group = n_out * nacc; p.w_scale = w_scale; p.x_scale = x_scale; p.x_scale_ld = x_scale_ld;
  p.out = out; p.out_ld = out_ld; p.out_f32 = out_f32; p.out_scale = out_scale; p.out_scale_ld = out_scale_ld;
  p.row_scale = row_scale; p.x_group_col = x_group_col; p.out_group_col = out_group_col;
  p.status = (OmniStatus*)status;
  if (x_ld <= 0) x_ld = K;
  const uint64_t x_cols = x_group_col > 0 ? (uint64_t)x_ld : (uint64_t)K;

  const int bk = (kind == 0) ? 64 : 128;
  CUtensorMap tw, tx;
  if (make_tmap_2d(&tw, w, esz, (uint64_t)G * p.w_rows_per_group, K, K, 128, bk, true)) return -10;
  if (x_group_col > 0 && (K % bk) != 0) return -6;  // a K tail would read the next group's columns
  if (make_tmap_2d(&tx, x, esz, (uint64_t)x_rows, x_cols, x_ld, bn, bk, true)) return -11;
  const int grid = sm_count();

#define OMNI_GEMM_CASE(KIND_, BN_, NACC_, EPI_) \
  if (kind == KIND_ && bn == BN_ && epi == EPI_) return launch_gemm<KIND_, BN_, NACC_, EPI_>(tw, tx, p, grid, stream);
  OMNI_GEMM_CASE(0, 32, 1, 0) OMNI_GEMM_CASE(0, 64, 1, 0) OMNI_GEMM_CASE(0, 128, 1, 0) OMNI_GEMM_CASE(0, 256, 1, 0)
  OMNI_GEMM_CASE(0, 32, 2, 1) OMNI_GEMM_CASE(0, 64, 2, 1) OMNI_GEMM_CASE(0, 128, 2, 1)
  OMNI_GEMM_CASE(1, 32, 1, 0) OMNI_GEMM_CASE(1, 64, 1, 0) OMNI_GEMM_CASE(1, 128, 1, 0)
  OMNI_GEMM_CASE(1, 32, 2, 1) OMNI_GEMM_CASE(1, 64, 2, 1)
  OMNI_GEMM_CASE(1, 32, 2, 2) OMNI_GEMM_CASE(1, 64, 2, 2)
#undef OMNI_GEMM_CASE
  return -20;
}
