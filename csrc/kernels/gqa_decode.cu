// Grouped-query attention decode over a paged K/V cache: one query token per request, D = 128, up to 16 query heads
// per KV head.
//
//   q        [B, Hq, 128] bf16
//   k_cache  [blocks, block_size, Hkv, 128] bf16 (v_cache alike)
//   out      [B, Hq, 128] bf16 = softmax(q k^T * scale) v over the first seq_lens[b] cache rows of request b
//
// The op is a stream over the cache (every K and V row is read once), so the kernel is built around keeping many
// independent 16 KB pieces of that stream in flight per SM.  grid (Hkv, splits, B), four warps per CTA; each warp owns a
// private 16 KB staging area and walks tiles of 32 keys on its own: it copies the tile's K and V rows with 16-byte
// cp.async (coalesced 256-byte rows, rows of keys past the end zero-filled), waits for them, and runs the tile's math
// on the tensor cores.  With three CTAs per SM twelve such streams run side by side, which covers the memory latency
// without any block-level synchronisation in the loop.
//
// Math per tile: the query heads that share the KV head are the rows of the MMA (mma.sync m16n8k16, rows past the
// group size are zero), S = Q K^T from ldmatrix fragments of the staged K rows, online softmax in registers (one row
// per lane quad), and O += P V with P taken straight from the S accumulators and V fragments from ldmatrix.trans.
// Staged rows are XOR-swizzled by 16-byte chunk so that both ldmatrix forms are free of bank conflicts.  The four
// warps' partial results are merged through shared memory at the end; a split-KV launch writes fp32 partials and
// log-sum-exps that a small second kernel combines.  This is a bandwidth-bound op on a few query rows, so the
// warp-level MMA is enough: the tensor pipe is idle most of the time either way.
//
// Reference counterpart: the paged decode attention of the GQA backend
// (omni/models/common/layers/attention/backend/attention.py:507-702).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace omni {

constexpr int GQ_D = 128;
constexpr int GQ_TILE = 32;                            // keys per warp tile
constexpr int GQ_ROW_BYTES = GQ_D * 2;                 // 256
constexpr int GQ_STAGE_BYTES = 2 * GQ_TILE * GQ_ROW_BYTES;   // K and V of one tile: 16 KB
constexpr int GQ_WARPS = 4;
constexpr int GQ_Q_BYTES = 16 * GQ_ROW_BYTES;          // 16 query rows (zero padded)
constexpr int GQ_SMEM = GQ_WARPS * GQ_STAGE_BYTES + GQ_Q_BYTES;
static_assert(GQ_WARPS * GQ_STAGE_BYTES >= GQ_WARPS * 16 * GQ_D * 4 + 2 * GQ_WARPS * 16 * 4,
              "the staging area is reused for the merge of the four warps");

__device__ __forceinline__ uint32_t gq_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t gq_swz(int row, int chunk) { return (uint32_t)(row * GQ_ROW_BYTES + ((chunk ^ (row & 7)) << 4)); }

__device__ __forceinline__ void gq_cp_async16(uint32_t dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;     // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void gq_cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

__device__ __forceinline__ void gq_ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void gq_ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void gq_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t gq_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(GQ_WARPS * 32, 3)
gqa_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                  const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ block_table, int bt_ld,
                  const int* __restrict__ seq_lens, int block_size, int Hq, int Hkv, float scale_log2, int splits,
                  float* __restrict__ o_part, float* __restrict__ lse_part, __nv_bfloat16* __restrict__ out) {
  extern __shared__ __align__(1024) uint8_t gq_smem[];
  const int hk = blockIdx.x, split = blockIdx.y, b = blockIdx.z;
  const int G = Hq / Hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int L = seq_lens[b];
  const int tiles = (L + GQ_TILE - 1) / GQ_TILE;
  const int tps = (tiles + splits - 1) / splits;
  const int t_begin = split * tps, t_end = min(tiles, t_begin + tps);

  uint8_t* stage = gq_smem + warp * GQ_STAGE_BYTES;           // [K tile 8 KB][V tile 8 KB]
  uint8_t* sq = gq_smem + GQ_WARPS * GQ_STAGE_BYTES;          // 16 x 128 bf16, swizzled like the tiles
  const uint32_t stage_k = gq_smem_u32(stage), stage_v = stage_k + GQ_TILE * GQ_ROW_BYTES, sq_addr = gq_smem_u32(sq);

  // query rows of this group (rows >= G are zero)
  for (int i = threadIdx.x; i < 16 * 16; i += blockDim.x) {
    const int row = i >> 4, chunk = i & 15;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (row < G) v = *reinterpret_cast<const uint4*>(q + ((size_t)b * Hq + hk * G + row) * GQ_D + chunk * 8);
    *reinterpret_cast<uint4*>(sq + gq_swz(row, chunk)) = v;
  }
  __syncthreads();
  // A fragments of Q for the eight 16-wide steps over the head dimension
  uint32_t qa[8][4];
  {
    const int row = ((lane >> 3) & 1) * 8 + (lane & 7), chalf = lane >> 4;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) gq_ldmatrix_x4(sq_addr + gq_swz(row, ks * 2 + chalf), qa[ks]);
  }

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[16][4];
#pragma unroll
  for (int j = 0; j < 16; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }

  for (int t = t_begin + warp; t < t_end; t += GQ_WARPS) {
    // ---- stage the tile: lane `r` knows where key row r of the tile lives
    const int my_key = t * GQ_TILE + lane;
    const bool my_valid = my_key < L;
    long long my_slot = 0;
    if (my_valid) my_slot = (long long)block_table[(size_t)b * bt_ld + my_key / block_size] * block_size + my_key % block_size;
#pragma unroll 4
    for (int it = 0; it < 16; ++it) {
      const int row = it * 2 + (lane >> 4), chunk = lane & 15;
      const long long slot = __shfl_sync(0xffffffffu, my_slot, row);
      const bool valid = __shfl_sync(0xffffffffu, (int)my_valid, row) != 0;
      const size_t off = ((size_t)slot * Hkv + hk) * GQ_D + chunk * 8;
      gq_cp_async16(stage_k + gq_swz(row, chunk), k_cache + off, valid);
      gq_cp_async16(stage_v + gq_swz(row, chunk), v_cache + off, valid);
    }
    gq_cp_async_wait_all();
    __syncwarp();

    // ---- S = Q K^T : four 8-key column tiles
    float s[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int krow = j * 8 + (lane & 7);
#pragma unroll
      for (int kp = 0; kp < 4; ++kp) {          // two 16-wide steps per ldmatrix.x4
        uint32_t kb[4];
        gq_ldmatrix_x4(stage_k + gq_swz(krow, kp * 4 + (lane >> 3)), kb);
        gq_mma(s[j], qa[2 * kp], kb[0], kb[1]);
        gq_mma(s[j], qa[2 * kp + 1], kb[2], kb[3]);
      }
    }
    // ---- online softmax: rows g = lane / 4 and g + 8; this lane holds 8 of the 32 scores of each
    const int key0 = t * GQ_TILE + (lane & 3) * 2;
    float mt[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key0 + j * 8 + (e & 1);
        const float v = key < L ? s[j][e] * scale_log2 : -INFINITY;
        s[j][e] = v;
        mt[e >> 1] = fmaxf(mt[e >> 1], v);
      }
    }
    float f[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mt[r] = fmaxf(mt[r], __shfl_xor_sync(0xffffffffu, mt[r], 1));
      mt[r] = fmaxf(mt[r], __shfl_xor_sync(0xffffffffu, mt[r], 2));
      const float m_new = fmaxf(m[r], mt[r]);
      f[r] = m_new == -INFINITY ? 1.f : exp2f(m[r] - m_new);
      m[r] = m_new;
    }
    float rs[2] = {0.f, 0.f};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float p = m[e >> 1] == -INFINITY ? 0.f : exp2f(s[j][e] - m[e >> 1]);
        s[j][e] = p;
        rs[e >> 1] += p;
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 1);
      rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 2);
      l[r] = l[r] * f[r] + rs[r];
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) { o[j][0] *= f[0]; o[j][1] *= f[0]; o[j][2] *= f[1]; o[j][3] *= f[1]; }
    // ---- O += P V : two 16-key steps, sixteen 8-wide output tiles
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
      uint32_t pa[4];
      pa[0] = gq_pack(s[2 * ks][0], s[2 * ks][1]);
      pa[1] = gq_pack(s[2 * ks][2], s[2 * ks][3]);
      pa[2] = gq_pack(s[2 * ks + 1][0], s[2 * ks + 1][1]);
      pa[3] = gq_pack(s[2 * ks + 1][2], s[2 * ks + 1][3]);
      const int vrow = ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
#pragma unroll
      for (int jp = 0; jp < 8; ++jp) {          // two output tiles per ldmatrix.x4.trans
        uint32_t vb[4];
        gq_ldmatrix_x4_trans(stage_v + gq_swz(vrow, jp * 2 + (lane >> 4)), vb);
        gq_mma(o[2 * jp], pa, vb[0], vb[1]);
        gq_mma(o[2 * jp + 1], pa, vb[2], vb[3]);
      }
    }
    __syncwarp();      // every lane is done with the staged tile before the next copies land
  }

  // ---- merge the four warps (staging memory is free now)
  __syncthreads();
  float* s_o = reinterpret_cast<float*>(gq_smem);                     // [4][16][128]
  float* s_m = s_o + GQ_WARPS * 16 * GQ_D;                            // [4][16]
  float* s_l = s_m + GQ_WARPS * 16;
  {
    const int g = lane >> 2, c = (lane & 3) * 2;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      float* r0 = s_o + ((size_t)warp * 16 + g) * GQ_D + j * 8 + c;
      float* r1 = s_o + ((size_t)warp * 16 + g + 8) * GQ_D + j * 8 + c;
      r0[0] = o[j][0]; r0[1] = o[j][1]; r1[0] = o[j][2]; r1[1] = o[j][3];
    }
    if ((lane & 3) == 0) {
      s_m[warp * 16 + g] = m[0]; s_m[warp * 16 + g + 8] = m[1];
      s_l[warp * 16 + g] = l[0]; s_l[warp * 16 + g + 8] = l[1];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * GQ_D; idx += blockDim.x) {
    const int g = idx / GQ_D, d = idx - g * GQ_D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < GQ_WARPS; ++w) mm = fmaxf(mm, s_m[w * 16 + g]);
    float ll = 0.f, acc = 0.f;
    if (mm > -INFINITY) {
#pragma unroll
      for (int w = 0; w < GQ_WARPS; ++w) {
        const float mw = s_m[w * 16 + g];
        const float fw = mw == -INFINITY ? 0.f : exp2f(mw - mm);
        ll += s_l[w * 16 + g] * fw;
        acc += s_o[((size_t)w * 16 + g) * GQ_D + d] * fw;
      }
    }
    const int hq = hk * G + g;
    if (splits == 1) {
      out[((size_t)b * Hq + hq) * GQ_D + d] = __float2bfloat16(ll > 0.f ? acc / ll : 0.f);
    } else {
      o_part[(((size_t)b * splits + split) * Hq + hq) * GQ_D + d] = ll > 0.f ? acc / ll : 0.f;
      if (d == 0) lse_part[((size_t)b * splits + split) * Hq + hq] = ll > 0.f ? mm + log2f(ll) : -INFINITY;
    }
  }
}

__global__ void gqa_combine_kernel(const float* __restrict__ o_part, const float* __restrict__ lse_part, int splits,
                                   int Hq, __nv_bfloat16* out) {
  const int bh = blockIdx.x;
  const int b = bh / Hq, h = bh - b * Hq;
  const int d = threadIdx.x;
  float mx = -INFINITY;
  for (int s = 0; s < splits; ++s) mx = fmaxf(mx, lse_part[((size_t)b * splits + s) * Hq + h]);
  float den = 0.f, acc = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float v = lse_part[((size_t)b * splits + s) * Hq + h];
    if (v == -INFINITY) continue;
    const float w = exp2f(v - mx);
    den += w;
    acc += w * o_part[(((size_t)b * splits + s) * Hq + h) * GQ_D + d];
  }
  out[(size_t)bh * GQ_D + d] = __float2bfloat16(den > 0.f ? acc / den : 0.f);
}

}  // namespace omni

using namespace omni;

extern "C" int omni_gqa_paged_decode(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                                     int bt_ld, const int* seq_lens, int B, int Hq, int Hkv, int D, int block_size,
                                     float scale, int splits, float* o_part, float* lse_part, void* out,
                                     cudaStream_t stream) {
  if (B <= 0) return 0;
  if (D != GQ_D || Hq % Hkv != 0 || Hq / Hkv > 16 || splits < 1) return -1;
  if (splits > 1 && (o_part == nullptr || lse_part == nullptr)) return -2;
  static bool configured[64] = {false};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    e = cudaFuncSetAttribute(gqa_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GQ_SMEM);
    if (e != cudaSuccess) return (int)e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  dim3 grid(Hkv, splits, B);
  gqa_decode_kernel<<<grid, GQ_WARPS * 32, GQ_SMEM, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache,
                                                             (const __nv_bfloat16*)v_cache, block_table, bt_ld, seq_lens,
                                                             block_size, Hq, Hkv, scale * 1.4426950408889634f, splits, o_part,
                                                             lse_part, (__nv_bfloat16*)out);
  e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  if (splits > 1) {
    gqa_combine_kernel<<<B * Hq, GQ_D, 0, stream>>>(o_part, lse_part, splits, Hq, (__nv_bfloat16*)out);
    e = cudaGetLastError();
  }
  return (int)e;
}
