// MLA absorbed-weight decode attention over a paged latent cache (tcgen05 + TMEM, sm_100a).
//
//   q      [Bq, H, 576]  bf16   absorbed query: 512 latent dims | 64 rope dims
//   cache  [slots, 576]  bf16   one "KV head": normalised latent c_kv (512) | roped k_pe (64); keys are
//                               the full 576-wide row, values are its first 512 entries
//   out    [Bq, H, 512]  bf16   softmax(q k^T * scale) v   (still in latent space; W_UV follows)
//
// Work split.  The q heads of one row are the UMMA M dimension (128 lanes, one head per TMEM lane and
// per softmax thread, so row max / row sum never leave the thread).  The fp32 output accumulator of 128
// heads x 512 dims would fill all of TMEM, so two CTAs (blockIdx.x = 0/1) each own 256 output dims;
// both compute the full score tile.  blockIdx.y splits the KV range (flash-decoding), blockIdx.z = q row.
//
// Per CTA: warp 0 = TMA producer, warp 1 = MMA issuer, warps 2..5 = softmax / correction / epilogue.
//   S = Q K^T     A = Q  (smem, K-major, 9 chunks of 64 dims)   B = KV tile (smem, K-major)      -> TMEM
//   P = softmax   written back to TMEM as packed bf16 (A operand of the second MMA)
//   O += P V      A = P  (TMEM)                                  B = KV tile (same smem, MN-major) -> TMEM
// Four of the nine 64-dim q chunks sit in shared memory, the other five in TMEM (as A operands), which
// leaves room for four KV stages.  KV tiles are 32 tokens; the chunks that only the score MMA reads (the other CTA's
// value dims and the rope dims) are released as soon as S is issued, the value chunks after P V.
// The running max is only raised when it grows by more than 2^8 (lazy rescale), so the O accumulator is
// rarely read back.
//
// Stands where the reference calls npu_fused_infer_attention_score on the absorbed path
// (omni/models/common/layers/attention/deepseek_mla.py:533-560, 625-650).
#include "../include/omni_ptx.cuh"
#include "../include/tma_host.h"

namespace omni {

struct MlaDecodeParams {
  int H;
  int block_size;
  const int* block_table;
  int bt_ld;
  const int* seq_lens;   // [Bq] visible kv tokens of each q row
  const int* q_to_seq;   // [Bq] block-table row of each q row, or null (identity)
  const __nv_bfloat16* q; // [Bq, H, 576] (also read directly for the chunks kept in TMEM)
  float scale_log2;      // softmax scale * log2(e)
  int num_splits;
  __nv_bfloat16* out;    // [Bq, H, 512]
  float* o_part;         // [Bq, splits, H, 512]
  float* lse_part;       // [Bq, splits, H]   (log2 domain)
  OmniStatus* status;
};

constexpr int MLA_TILE = 32;
constexpr int MLA_CHUNK_BYTES = MLA_TILE * 128;       // 32 tokens x 64 dims bf16
constexpr int MLA_STAGE_BYTES = 9 * MLA_CHUNK_BYTES;  // 36 KB
constexpr int MLA_Q_CHUNK = 128 * 128;                // 128 heads x 64 dims bf16
constexpr int MLA_Q_BYTES = 9 * MLA_Q_CHUNK;          // 144 KB
constexpr int MLA_QS = 4;                             // q chunks 0..3 live in shared memory,
constexpr int MLA_QT = 5;                             // chunks 4..8 (latent dims 256..511 + rope) in TMEM
constexpr int MLA_STAGES = 4;
constexpr int MLA_SMEM = MLA_QS * MLA_Q_CHUNK + MLA_STAGES * MLA_STAGE_BYTES + 1024 /*barriers*/ + 1024 /*align*/;
constexpr int MLA_THREADS = 192;
// TMEM columns: O accumulator | two S tiles | two packed-bf16 P tiles | five packed-bf16 q chunks
constexpr int TM_O = 0, TM_S = 256, TM_P = 320, TM_Q = 352, TM_COLS = 512;

enum { MS_Q = 1, MS_KA_EMPTY, MS_KB_EMPTY, MS_KA_FULL, MS_KB_FULL, MS_P_FULL, MS_S_FULL, MS_O_DONE, MS_QT };

__device__ __forceinline__ void umma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_st_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

__global__ void __launch_bounds__(MLA_THREADS, 1)
mla_decode_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_kv,
                  const MlaDecodeParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sq = smem;
  uint8_t* skv = smem + MLA_QS * MLA_Q_CHUNK;
  uint64_t* bars = (uint64_t*)(skv + MLA_STAGES * MLA_STAGE_BYTES);
  uint64_t* q_full = bars;                          // 1
  uint64_t* ka_full = bars + 1;                     // STAGES
  uint64_t* ka_empty = ka_full + MLA_STAGES;
  uint64_t* kb_full = ka_empty + MLA_STAGES;
  uint64_t* kb_empty = kb_full + MLA_STAGES;
  uint64_t* s_full = kb_empty + MLA_STAGES;         // 2
  uint64_t* p_full = s_full + 2;                    // 2
  uint64_t* o_done = p_full + 2;                    // 1
  uint64_t* o_final = o_done + 1;                   // 1: all P V of this CTA retired
  uint64_t* qt_full = o_final + 1;                  // 1: q chunks written to TMEM
  uint32_t* tmem_slot = (uint32_t*)(qt_full + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int half = blockIdx.x;   // which 256 output dims
  const int split = blockIdx.y;
  const int bq = blockIdx.z;

  const int kv_len = p.seq_lens[bq];
  const int tiles_total = (kv_len + MLA_TILE - 1) / MLA_TILE;
  const int tps = (tiles_total + p.num_splits - 1) / p.num_splits;
  const int tile_begin = split * tps;
  const int tile_end = min(tiles_total, tile_begin + tps);
  const int n = max(0, tile_end - tile_begin);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < MLA_STAGES; ++s) {
      mbar_init(&ka_full[s], 1);
      mbar_init(&ka_empty[s], 1);
      mbar_init(&kb_full[s], 1);
      mbar_init(&kb_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 4);
    }
    mbar_init(o_done, 1);
    mbar_init(o_final, 1);
    mbar_init(qt_full, 4);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // chunks 0..7 = latent dims 64c..64c+63, chunk 8 = rope dims.  Group B = this CTA's value chunks.
  const int vb = half * 4;  // first value chunk of this CTA

  if (n > 0) {
    if (warp == 0) {
      if (lane == 0) {
        tma_prefetch_desc(&tmap_q);
        tma_prefetch_desc(&tmap_kv);
        mbar_expect_tx(q_full, MLA_QS * MLA_Q_CHUNK);
        for (int c = 0; c < MLA_QS; ++c) tma_load_2d(sq + c * MLA_Q_CHUNK, &tmap_q, q_full, c * 64, bq * p.H);
        const int seq = p.q_to_seq ? p.q_to_seq[bq] : bq;
        const int* bt = p.block_table + (size_t)seq * p.bt_ld;
        for (int i = 0; i < n; ++i) {
          const int st = i % MLA_STAGES;
          const uint32_t ph = (i / MLA_STAGES) & 1;
          const int tok0 = (tile_begin + i) * MLA_TILE;
          const int page = bt[tok0 / p.block_size];
          const int row = page * p.block_size + tok0 % p.block_size;
          uint8_t* base = skv + st * MLA_STAGE_BYTES;
          if (!mbar_wait(&ka_empty[st], ph ^ 1, abort_flag, p.status, MS_KA_EMPTY, i)) break;
          mbar_expect_tx(&ka_full[st], 5 * MLA_CHUNK_BYTES);
          for (int c = 0; c < 9; ++c)
            if (c < vb || c >= vb + 4) tma_load_2d(base + c * MLA_CHUNK_BYTES, &tmap_kv, &ka_full[st], c * 64, row);
          if (!mbar_wait(&kb_empty[st], ph ^ 1, abort_flag, p.status, MS_KB_EMPTY, i)) break;
          mbar_expect_tx(&kb_full[st], 4 * MLA_CHUNK_BYTES);
          for (int c = vb; c < vb + 4; ++c)
            tma_load_2d(base + c * MLA_CHUNK_BYTES, &tmap_kv, &kb_full[st], c * 64, row);
        }
      }
    } else if (warp == 1) {
      if (lane == 0) {
        constexpr uint32_t idesc_qk = umma_idesc(128, MLA_TILE, 1, 1, 0, 0);
        constexpr uint32_t idesc_pv = umma_idesc(128, 256, 1, 1, 0, 1);
        bool ok = mbar_wait(q_full, 0, abort_flag, p.status, MS_Q, 0);
        if (ok) ok = mbar_wait(qt_full, 0, abort_flag, p.status, MS_QT, 0);
        tc_fence_after();
        // q chunk c times kv chunk c of the staged tile; q comes from shared memory or from TMEM
        auto qk_chunk = [&](uint32_t d, uint32_t kbase, int c, uint32_t& accum) {
          const uint64_t bd = umma_desc_kmajor_sw128(kbase + c * MLA_CHUNK_BYTES);
          if (c < MLA_QS) {
            const uint64_t ad = umma_desc_kmajor_sw128(smem_u32(sq) + c * MLA_Q_CHUNK);
#pragma unroll
            for (int k = 0; k < 4; ++k) { umma_bf16(d, ad + 2 * k, bd + 2 * k, idesc_qk, accum); accum = 1; }
          } else {
            const uint32_t at = tmem_base + TM_Q + (c - MLA_QS) * 32;
#pragma unroll
            for (int k = 0; k < 4; ++k) { umma_bf16_ts(d, at + 8 * k, bd + 2 * k, idesc_qk, accum); accum = 1; }
          }
        };
        auto issue_qk = [&](int j) -> bool {
          const int st = j % MLA_STAGES;
          const uint32_t ph = (j / MLA_STAGES) & 1;
          const uint32_t kbase = smem_u32(skv + st * MLA_STAGE_BYTES);
          const uint32_t d = tmem_base + TM_S + (j & 1) * MLA_TILE;
          uint32_t accum = 0;
          if (!mbar_wait(&ka_full[st], ph, abort_flag, p.status, MS_KA_FULL, j)) return false;
          tc_fence_after();
          for (int c = 0; c < 9; ++c) {
            if (c >= vb && c < vb + 4) continue;
            qk_chunk(d, kbase, c, accum);
          }
          umma_commit(&ka_empty[st]);
          if (!mbar_wait(&kb_full[st], ph, abort_flag, p.status, MS_KB_FULL, j)) return false;
          tc_fence_after();
          for (int c = vb; c < vb + 4; ++c) qk_chunk(d, kbase, c, accum);
          umma_commit(&s_full[j & 1]);
          return true;
        };
        if (ok) ok = issue_qk(0);
        if (ok && n > 1) ok = issue_qk(1);
        for (int i = 0; i < n && ok; ++i) {
          const int st = i % MLA_STAGES;
          if (!mbar_wait(&p_full[i & 1], (i >> 1) & 1, abort_flag, p.status, MS_P_FULL, i)) { ok = false; break; }
          tc_fence_after();
          const uint32_t vbase = smem_u32(skv + st * MLA_STAGE_BYTES) + vb * MLA_CHUNK_BYTES;
#pragma unroll
          for (int k = 0; k < MLA_TILE / 16; ++k) {
            // 16 tokens per MMA: two 8-token groups of 1024 B; dims advance by whole 4 KB chunks
            const uint64_t bd = umma_desc_mnmajor_sw128(vbase + k * 2048, MLA_CHUNK_BYTES, 1024);
            umma_bf16_ts(tmem_base + TM_O, tmem_base + TM_P + (i & 1) * (MLA_TILE / 2) + k * 8, bd, idesc_pv,
                         (i > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&kb_empty[st]);
          umma_commit(o_done);
          if (i == n - 1) umma_commit(o_final);
          if (i + 2 < n) ok = issue_qk(i + 2);
        }
      }
    } else {
      // ------------------------------------------------------------ softmax / correction / epilogue
      const int qd = warp & 3;
      const int row = qd * 32 + lane;  // head
      const uint32_t lane_addr = tmem_base + ((uint32_t)(qd * 32) << 16);
      float m = -INFINITY, l = 0.f;
      bool ok = true;
      // this head's q values for latent dims 256..511 and the rope dims go to TMEM as packed bf16 pairs
      {
        const uint4* qsrc = reinterpret_cast<const uint4*>(p.q + ((size_t)bq * p.H + row) * 576 + MLA_QS * 64);
        const bool row_ok = row < p.H;
#pragma unroll 1
        for (int c = 0; c < MLA_QT; ++c) {
          uint32_t v[32];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint4 x = row_ok ? __ldg(qsrc + c * 8 + j) : make_uint4(0, 0, 0, 0);
            v[4 * j] = x.x; v[4 * j + 1] = x.y; v[4 * j + 2] = x.z; v[4 * j + 3] = x.w;
          }
          tmem_st_x32(lane_addr + TM_Q + c * 32, v);
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(qt_full);
      }
      for (int i = 0; i < n; ++i) {
        const int st = i & 1;
        if (!mbar_wait(&s_full[st], (i >> 1) & 1, abort_flag, p.status, MS_S_FULL, i)) { ok = false; break; }
        tc_fence_after();
        uint32_t sv[32];
        tmem_ld_x32(lane_addr + TM_S + st * MLA_TILE, sv);
        tmem_ld_wait();
        const int valid = kv_len - (tile_begin + i) * MLA_TILE;  // >= 1
        float s[32];
        float mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          s[j] = (j < valid) ? __uint_as_float(sv[j]) * p.scale_log2 : -INFINITY;
          mx = fmaxf(mx, s[j]);
        }
        const float m_new = fmaxf(m, mx);
        const bool grow = (m_new - m) > 8.0f;  // also true on the first tile (m = -inf)
        if (i == 0) {
          m = m_new;
        } else if (__any_sync(0xffffffffu, grow)) {
          if (!mbar_wait(o_done, (i - 1) & 1, abort_flag, p.status, MS_O_DONE, i)) { ok = false; break; }
          tc_fence_after();
          const float f = grow ? exp2f(m - m_new) : 1.0f;
          if (grow) { l *= f; m = m_new; }
#pragma unroll 1
          for (int c = 0; c < 256; c += 32) {
            uint32_t ov[32];
            tmem_ld_x32(lane_addr + TM_O + c, ov);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) ov[j] = __float_as_uint(__uint_as_float(ov[j]) * f);
            tmem_st_x32(lane_addr + TM_O + c, ov);
          }
          tmem_st_wait();
        }
        uint32_t pk[16];
        float rs = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float p0 = exp2f(s[2 * j] - m), p1 = exp2f(s[2 * j + 1] - m);
          rs += p0 + p1;
          __nv_bfloat162 h2 = __floats2bfloat162_rn(p0, p1);
          pk[j] = *reinterpret_cast<uint32_t*>(&h2);
        }
        l += rs;
        tmem_st_x16(lane_addr + TM_P + st * (MLA_TILE / 2), pk);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[st]);
      }
      // o_done flips once per tile and is only sampled when a rescale is needed, so its parity cannot
      // tell "last tile retired" from "two tiles behind"; the single-use o_final barrier can.
      if (ok) ok = mbar_wait(o_final, 0, abort_flag, p.status, MS_O_DONE, n);
      if (ok) {
        tc_fence_after();
        const float inv_l = 1.0f / l;
        const bool row_ok = row < p.H;
        if (p.num_splits == 1) {
          __nv_bfloat16* orow = p.out + ((size_t)bq * p.H + row) * 512 + half * 256;
#pragma unroll 1
          for (int c = 0; c < 256; c += 32) {
            uint32_t ov[32];
            tmem_ld_x32(lane_addr + TM_O + c, ov);
            tmem_ld_wait();
            if (row_ok) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                __nv_bfloat16 o8[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) o8[e] = __float2bfloat16(__uint_as_float(ov[j + e]) * inv_l);
                *reinterpret_cast<uint4*>(orow + c + j) = *reinterpret_cast<uint4*>(o8);
              }
            }
          }
        } else {
          float* orow = p.o_part + (((size_t)bq * p.num_splits + split) * p.H + row) * 512 + half * 256;
#pragma unroll 1
          for (int c = 0; c < 256; c += 32) {
            uint32_t ov[32];
            tmem_ld_x32(lane_addr + TM_O + c, ov);
            tmem_ld_wait();
            if (row_ok) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                float4 o4 = make_float4(__uint_as_float(ov[j]) * inv_l, __uint_as_float(ov[j + 1]) * inv_l,
                                        __uint_as_float(ov[j + 2]) * inv_l, __uint_as_float(ov[j + 3]) * inv_l);
                *reinterpret_cast<float4*>(orow + c + j) = o4;
              }
            }
          }
          if (half == 0 && row_ok)
            p.lse_part[((size_t)bq * p.num_splits + split) * p.H + row] = m + log2f(l);
        }
      }
    }
  } else if (warp >= 2) {
    // empty KV range for this split (or an empty / padding row): neutral partial result
    const int row = (warp & 3) * 32 + lane;
    if (row < p.H) {
      if (p.num_splits == 1) {
        __nv_bfloat16* orow = p.out + ((size_t)bq * p.H + row) * 512 + half * 256;
        for (int c = 0; c < 256; c += 8) *reinterpret_cast<uint4*>(orow + c) = make_uint4(0, 0, 0, 0);
      } else {
        float* orow = p.o_part + (((size_t)bq * p.num_splits + split) * p.H + row) * 512 + half * 256;
        for (int c = 0; c < 256; c += 4) *reinterpret_cast<float4*>(orow + c) = make_float4(0.f, 0.f, 0.f, 0.f);
        if (half == 0) p.lse_part[((size_t)bq * p.num_splits + split) * p.H + row] = -INFINITY;
      }
    }
  }

  if (*abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TM_COLS);
  }
}

// out[bq, h, :] = sum_s w_s * o_part[bq, s, h, :],  w_s = 2^(lse_s - max) / sum
__global__ void mla_combine_kernel(const float* __restrict__ o_part, const float* __restrict__ lse_part,
                                   int splits, int H, __nv_bfloat16* out) {
  const int bh = blockIdx.x;  // bq * H + h
  const int bq = bh / H, h = bh - bq * H;
  float mx = -INFINITY;
  for (int s = 0; s < splits; ++s) mx = fmaxf(mx, lse_part[((size_t)bq * splits + s) * H + h]);
  float den = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float v = lse_part[((size_t)bq * splits + s) * H + h];
    den += (v == -INFINITY) ? 0.f : exp2f(v - mx);
  }
  const float inv = den > 0.f ? 1.f / den : 0.f;
  for (int c = threadIdx.x * 4; c < 512; c += blockDim.x * 4) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < splits; ++s) {
      const float v = lse_part[((size_t)bq * splits + s) * H + h];
      if (v == -INFINITY) continue;
      const float w = exp2f(v - mx) * inv;
      const float4 o = *reinterpret_cast<const float4*>(o_part + (((size_t)bq * splits + s) * H + h) * 512 + c);
      acc.x += w * o.x; acc.y += w * o.y; acc.z += w * o.z; acc.w += w * o.w;
    }
    __nv_bfloat16 o4[4] = {__float2bfloat16(acc.x), __float2bfloat16(acc.y), __float2bfloat16(acc.z),
                           __float2bfloat16(acc.w)};
    *reinterpret_cast<uint2*>(out + (size_t)bh * 512 + c) = *reinterpret_cast<uint2*>(o4);
  }
}

}  // namespace omni

using namespace omni;

// Scratch needed for num_splits > 1: o_part = Bq*splits*H*512 floats, lse_part = Bq*splits*H floats.
extern "C" int omni_mla_decode(const void* q, const void* cache, int cache_ld, long long num_slots,
                               const int* block_table, int bt_ld, const int* seq_lens, const int* q_to_seq, int Bq,
                               int H, int block_size, float scale, int num_splits, void* out, float* o_part,
                               float* lse_part, void* status, cudaStream_t stream) {
  if (Bq <= 0) return 0;
  if (H < 1 || H > 128) return -1;
  if (block_size % MLA_TILE != 0) return -2;
  if (num_splits < 1) return -3;
  if (num_splits > 1 && (o_part == nullptr || lse_part == nullptr)) return -4;
  CUtensorMap tq, tkv;
  if (make_tmap_2d(&tq, q, 2, (uint64_t)Bq * H, 576, 576, 128, 64, true)) return -10;
  if (make_tmap_2d(&tkv, cache, 2, (uint64_t)num_slots, 576, cache_ld, MLA_TILE, 64, true)) return -11;
  MlaDecodeParams p;
  p.q = (const __nv_bfloat16*)q; p.H = H; p.block_size = block_size; p.block_table = block_table; p.bt_ld = bt_ld; p.seq_lens = seq_lens;
  p.q_to_seq = q_to_seq; p.scale_log2 = scale * 1.4426950408889634f; p.num_splits = num_splits;
  p.out = (__nv_bfloat16*)out; p.o_part = o_part; p.lse_part = lse_part; p.status = (OmniStatus*)status;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(mla_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, MLA_SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(2, num_splits, Bq);
  mla_decode_kernel<<<grid, MLA_THREADS, MLA_SMEM, stream>>>(tq, tkv, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  if (num_splits > 1) {
    mla_combine_kernel<<<Bq * H, 128, 0, stream>>>(o_part, lse_part, num_splits, H, (__nv_bfloat16*)out);
    e = cudaGetLastError();
  }
  return (int)e;
}
