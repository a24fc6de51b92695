// Variable-length causal attention for prefill (tcgen05 + TMEM) and GQA paged decode.
//
// omni_fmha_varlen: one CTA per (128-query tile, request, q head).
//   S = Q K^T     A = Q tile (smem, K-major, 64-dim chunks)   B = K tile of 64 keys (smem, K-major)
//   P = softmax   kept in TMEM as packed bf16                  (thread = query row: no cross-thread reductions)
//   O += P V      A = P (TMEM)                                 B = V tile (smem, MN-major), 128 output dims
// The key dimension may come from two tensors: `k` (per kv head) and `k2` (shared by all heads).  That is how
// MLA prefill runs without materialising [k_nope | k_pe]: k/v are column slices of the kv_b_proj output,
// k2 is the roped k_pe slice of the latent rows.  GQA (Qwen) uses k only, with q heads mapped to kv heads.
// Causal mask is aligned to the end of the key range (query i of a request with Lq queries and Lk keys sees
// keys <= Lk - Lq + i), which also covers chunked prefill and prefix-cache hits.
//
// The paged decode of the GQA models (one query token per request) is a separate kernel: gqa_decode.cu.
//
// Reference call sites: npu_fused_infer_attention_score / npu_fusion_attention
// (omni/models/common/layers/attention/deepseek_mla.py:386-400, omni/models/common/layers/attention/backend/attention.py:590-666).
#include "../include/omni_ptx.cuh"
#include "../include/tma_host.h"

namespace omni {

struct FmhaParams {
  const int* cu_q;   // [B+1]
  const int* cu_k;   // [B+1]
  int Hq, Hkv;
  int q_head_stride, k_head_stride, v_head_stride;  // in elements (column offset per head)
  int v_col0, k2_col0;
  int nk1, nk2;      // number of 64-wide key chunks taken from k and from k2
  float scale_log2;
  int causal;
  __nv_bfloat16* out;  // [Tq, Hq * 128]
  OmniStatus* status;
};

constexpr int FM_BQ = 128, FM_BK = 64, FM_DV = 128;
constexpr int FM_QCHUNK = FM_BQ * 128;          // 16 KB
constexpr int FM_KCHUNK = FM_BK * 128;          // 8 KB
constexpr int FM_MAXC = 3;                      // up to 192 qk dims
constexpr int FM_STAGES = 3;
constexpr int FM_K_STAGE = FM_MAXC * FM_KCHUNK; // 24 KB
constexpr int FM_V_STAGE = 2 * FM_KCHUNK;       // 16 KB
constexpr int FM_SMEM = FM_MAXC * FM_QCHUNK + FM_STAGES * (FM_K_STAGE + FM_V_STAGE) + 1024 + 1024;
constexpr int FM_THREADS = 192;
constexpr int FT_O = 0, FT_S = 128, FT_P = 256, FT_COLS = 512;

__device__ __forceinline__ void fm_umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__global__ void __launch_bounds__(FM_THREADS, 1)
fmha_varlen_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                   const __grid_constant__ CUtensorMap tmap_k2, const __grid_constant__ CUtensorMap tmap_v,
                   const FmhaParams p) {
  const int b = blockIdx.y, h = blockIdx.z;
  const int q_begin = p.cu_q[b], q_end = p.cu_q[b + 1];
  const int k_begin = p.cu_k[b], k_end = p.cu_k[b + 1];
  const int Lq = q_end - q_begin, Lk = k_end - k_begin;
  const int q0 = blockIdx.x * FM_BQ;
  if (q0 >= Lq) return;  // uniform for the whole CTA, before any barrier / TMEM use
  const int ctx = Lk - Lq;
  const int hk = h / (p.Hq / p.Hkv);
  const int nc = p.nk1 + p.nk2;
  // keys this tile can see
  int k_hi = p.causal ? min(Lk, ctx + q0 + FM_BQ) : Lk;
  const int n = (k_hi + FM_BK - 1) / FM_BK;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sq = smem;
  uint8_t* sk = smem + FM_MAXC * FM_QCHUNK;
  uint8_t* sv = sk + FM_STAGES * FM_K_STAGE;
  uint64_t* bars = (uint64_t*)(sv + FM_STAGES * FM_V_STAGE);
  uint64_t* q_full = bars;                       // 1
  uint64_t* k_full = bars + 1;                   // STAGES
  uint64_t* k_empty = k_full + FM_STAGES;
  uint64_t* v_full = k_empty + FM_STAGES;
  uint64_t* v_empty = v_full + FM_STAGES;
  uint64_t* s_full = v_empty + FM_STAGES;        // 2
  uint64_t* p_full = s_full + 2;                 // 2
  uint64_t* o_done = p_full + 2;                 // 1
  uint64_t* o_final = o_done + 1;                // 1
  uint32_t* tmem_slot = (uint32_t*)(o_final + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < FM_STAGES; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) { mbar_init(&s_full[s], 1); mbar_init(&p_full[s], 4); }
    mbar_init(o_done, 1);
    mbar_init(o_final, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, FT_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, nc * FM_QCHUNK);
      for (int c = 0; c < nc; ++c)
        tma_load_2d(sq + c * FM_QCHUNK, &tmap_q, q_full, h * p.q_head_stride + c * 64, q_begin + q0);
      for (int i = 0; i < n; ++i) {
        const int st = i % FM_STAGES;
        const uint32_t ph = (i / FM_STAGES) & 1;
        const int row = k_begin + i * FM_BK;
        if (!mbar_wait(&k_empty[st], ph ^ 1, abort_flag, p.status, 11, i)) break;
        mbar_expect_tx(&k_full[st], nc * FM_KCHUNK);
        for (int c = 0; c < p.nk1; ++c)
          tma_load_2d(sk + st * FM_K_STAGE + c * FM_KCHUNK, &tmap_k, &k_full[st], hk * p.k_head_stride + c * 64, row);
        for (int c = 0; c < p.nk2; ++c)
          tma_load_2d(sk + st * FM_K_STAGE + (p.nk1 + c) * FM_KCHUNK, &tmap_k2, &k_full[st], p.k2_col0 + c * 64, row);
        if (!mbar_wait(&v_empty[st], ph ^ 1, abort_flag, p.status, 12, i)) break;
        mbar_expect_tx(&v_full[st], 2 * FM_KCHUNK);
        for (int c = 0; c < 2; ++c)
          tma_load_2d(sv + st * FM_V_STAGE + c * FM_KCHUNK, &tmap_v, &v_full[st],
                      hk * p.v_head_stride + p.v_col0 + c * 64, row);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc(128, FM_BK, 1, 1, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc(128, FM_DV, 1, 1, 0, 1);
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, 13, 0);
      auto issue_qk = [&](int j) -> bool {
        const int st = j % FM_STAGES;
        if (!mbar_wait(&k_full[st], (j / FM_STAGES) & 1, abort_flag, p.status, 14, j)) return false;
        tc_fence_after();
        const uint32_t d = tmem_base + FT_S + (j & 1) * FM_BK;
        uint32_t accum = 0;
        for (int c = 0; c < nc; ++c) {
          const uint64_t ad = umma_desc_kmajor_sw128(smem_u32(sq) + c * FM_QCHUNK);
          const uint64_t bd = umma_desc_kmajor_sw128(smem_u32(sk) + st * FM_K_STAGE + c * FM_KCHUNK);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            umma_bf16(d, ad + 2 * k, bd + 2 * k, idesc_qk, accum);
            accum = 1;
          }
        }
        umma_commit(&k_empty[st]);
        umma_commit(&s_full[j & 1]);
        return true;
      };
      if (ok) ok = issue_qk(0);
      if (ok && n > 1) ok = issue_qk(1);
      for (int i = 0; i < n && ok; ++i) {
        const int st = i % FM_STAGES;
        if (!mbar_wait(&p_full[i & 1], (i >> 1) & 1, abort_flag, p.status, 15, i)) { ok = false; break; }
        if (!mbar_wait(&v_full[st], (i / FM_STAGES) & 1, abort_flag, p.status, 16, i)) { ok = false; break; }
        tc_fence_after();
        const uint32_t vbase = smem_u32(sv) + st * FM_V_STAGE;
#pragma unroll
        for (int k = 0; k < FM_BK / 16; ++k) {
          const uint64_t bd = umma_desc_mnmajor_sw128(vbase + k * 2048, FM_KCHUNK, 1024);
          fm_umma_ts(tmem_base + FT_O, tmem_base + FT_P + (i & 1) * (FM_BK / 2) + k * 8, bd, idesc_pv,
                     (i > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&v_empty[st]);
        umma_commit(o_done);
        if (i == n - 1) umma_commit(o_final);
        if (i + 2 < n) ok = issue_qk(i + 2);
      }
    }
  } else {
    const int qd = warp & 3;
    const int row = qd * 32 + lane;          // query row inside the tile
    const uint32_t lane_addr = tmem_base + ((uint32_t)(qd * 32) << 16);
    const int q_pos = ctx + q0 + row;        // last key index this row may see (causal)
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int i = 0; i < n; ++i) {
      if (!mbar_wait(&s_full[i & 1], (i >> 1) & 1, abort_flag, p.status, 17, i)) { ok = false; break; }
      tc_fence_after();
      const int kbase = i * FM_BK;
      int lim = Lk - kbase;                        // keys beyond the request end are masked
      if (p.causal) lim = min(lim, q_pos - kbase + 1);
      float s[FM_BK];
      float mx = -INFINITY;
#pragma unroll
      for (int c0 = 0; c0 < FM_BK; c0 += 32) {
        uint32_t sv32[32];
        tmem_ld_x32(lane_addr + FT_S + (i & 1) * FM_BK + c0, sv32);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          s[c0 + j] = (c0 + j < lim) ? __uint_as_float(sv32[j]) * p.scale_log2 : -INFINITY;
          mx = fmaxf(mx, s[c0 + j]);
        }
      }
      // rows past the end of the request (and, never in practice, fully masked rows) stay finite
      const float m_cand = fmaxf(m, mx);
      const float m_new = (m_cand == -INFINITY) ? 0.f : m_cand;
      const bool grow = (m_new - m) > 8.0f;
      if (i == 0) {
        m = m_new;
      } else if (__any_sync(0xffffffffu, grow)) {
        if (!mbar_wait(o_done, (i - 1) & 1, abort_flag, p.status, 18, i)) { ok = false; break; }
        tc_fence_after();
        const float f = grow ? exp2f(m - m_new) : 1.0f;
        if (grow) { l *= f; m = m_new; }
#pragma unroll 1
        for (int c = 0; c < FM_DV; c += 32) {
          uint32_t ov[32];
          tmem_ld_x32(lane_addr + FT_O + c, ov);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) ov[j] = __float_as_uint(__uint_as_float(ov[j]) * f);
          tmem_st_x32(lane_addr + FT_O + c, ov);
        }
        tmem_st_wait();
      }
      uint32_t pk[32];
      float rs = 0.f;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float p0 = exp2f(s[2 * j] - m), p1 = exp2f(s[2 * j + 1] - m);
        rs += p0 + p1;
        __nv_bfloat162 h2 = __floats2bfloat162_rn(p0, p1);
        pk[j] = *reinterpret_cast<uint32_t*>(&h2);
      }
      l += rs;
      tmem_st_x32(lane_addr + FT_P + (i & 1) * (FM_BK / 2), pk);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[i & 1]);
    }
    if (ok) ok = mbar_wait(o_final, 0, abort_flag, p.status, 19, n);
    if (ok) {
      tc_fence_after();
      const bool row_ok = (q0 + row) < Lq;
      const float inv_l = l > 0.f ? 1.0f / l : 0.f;
      __nv_bfloat16* orow = p.out + ((size_t)(q_begin + q0 + row) * p.Hq + h) * FM_DV;
#pragma unroll 1
      for (int c = 0; c < FM_DV; c += 32) {
        uint32_t ov[32];
        tmem_ld_x32(lane_addr + FT_O + c, ov);
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
    }
  }

  if (*abort_flag) {
    if (threadIdx.x == 0) report_abort(abort_flag, p.status);
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, FT_COLS);
  }
}

}  // namespace omni

using namespace omni;

// q/k/k2/v are 2-D row-major bf16 matrices given by (pointer, rows, row pitch in elements, columns).
extern "C" int omni_fmha_varlen(const void* q, long long q_rows, int q_ld, int q_cols, const void* k, long long k_rows,
                                int k_ld, int k_cols, const void* k2, int k2_ld, int k2_cols, const void* v, int v_ld,
                                int v_cols, const int* cu_q, const int* cu_k, int B, int max_q, int Hq, int Hkv,
                                int q_head_stride, int k_head_stride, int v_head_stride, int v_col0, int k2_col0,
                                int d_k1, int d_k2, int d_v, float scale, int causal, void* out, void* status,
                                cudaStream_t stream) {
  if (B <= 0 || max_q <= 0) return 0;
  if (d_v != 128 || d_k1 % 64 != 0 || d_k2 % 64 != 0 || (d_k1 + d_k2) > 64 * FM_MAXC) return -1;
  if (Hq % Hkv != 0) return -2;
  CUtensorMap tq, tk, tk2, tv;
  if (make_tmap_2d(&tq, q, 2, (uint64_t)q_rows, q_cols, q_ld, FM_BQ, 64, true)) return -10;
  if (make_tmap_2d(&tk, k, 2, (uint64_t)k_rows, k_cols, k_ld, FM_BK, 64, true)) return -11;
  if (d_k2 > 0) {
    if (make_tmap_2d(&tk2, k2, 2, (uint64_t)k_rows, k2_cols, k2_ld, FM_BK, 64, true)) return -12;
  } else {
    tk2 = tk;
  }
  if (make_tmap_2d(&tv, v, 2, (uint64_t)k_rows, v_cols, v_ld, FM_BK, 64, true)) return -13;
  FmhaParams p;
  p.cu_q = cu_q; p.cu_k = cu_k; p.Hq = Hq; p.Hkv = Hkv; p.q_head_stride = q_head_stride;
  p.k_head_stride = k_head_stride; p.v_head_stride = v_head_stride; p.v_col0 = v_col0; p.k2_col0 = k2_col0;
  p.nk1 = d_k1 / 64; p.nk2 = d_k2 / 64; p.scale_log2 = scale * 1.4426950408889634f; p.causal = causal;
  p.out = (__nv_bfloat16*)out; p.status = (OmniStatus*)status;
  static bool configured[64] = {false};
  if (int e = ensure_dyn_smem((const void*)fmha_varlen_kernel, FM_SMEM, configured)) return e;
  dim3 grid((max_q + FM_BQ - 1) / FM_BQ, B, Hq);
  fmha_varlen_kernel<<<grid, FM_THREADS, FM_SMEM, stream>>>(tq, tk, tk2, tv, p);
  return (int)cudaGetLastError();
}
