// Bandwidth-bound elementwise / row kernels around attention:
//   omni_rmsnorm            residual add + RMSNorm (+ e4m3 1x128 block quantisation of the output)
//   omni_quant_fp8_block    bf16 [T,K] -> e4m3 + per-(row,128) scales (K-block-major scale layout)
//   omni_mla_kv_rope_cache  latent [T,576]: RMSNorm(512) | interleaved RoPE(64) -> paged latent cache,
//                           and RoPE of the q rope slice in the same launch
//   omni_rope_qk_cache      GQA: optional per-head RMSNorm, neox RoPE on q/k, K/V scatter into the paged cache
//   omni_silu_mul           SwiGLU for the unfused paths
// They stand where the reference calls npu_add_rms_norm / npu_rms_norm / npu_dynamic_quant
// (omni/models/common/layers/layernorm.py:13-31), npu_kv_rmsnorm_rope_cache and npu_interleave_rope
// (omni/models/common/layers/attention/deepseek_mla.py:311-340, 493-526), npu_apply_rotary_pos_emb and
// _npu_reshape_and_cache (omni/models/common/layers/attention/backend/attention.py:560-580).
#include "../include/omni_ptx.cuh"

namespace omni {

union Pack8 {
  uint4 u;
  __nv_bfloat16 h[8];
};

// One CTA per row.  Each thread owns up to VPT vectors of 8 bf16.
template <int VPT>
__global__ void __launch_bounds__(256) rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* residual,
                                                      const __nv_bfloat16* __restrict__ weight, __nv_bfloat16* out,
                                                      uint8_t* out_q, float* out_scale, int out_scale_ld, int H,
                                                      int x_ld, float eps) {
  const int row = blockIdx.x;
  const int nvec = H >> 3;
  const __nv_bfloat16* xr = x + (size_t)row * x_ld;
  float v[VPT][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int vi = threadIdx.x + i * 256;
    if (vi < nvec) {
      Pack8 a;
      a.u = *reinterpret_cast<const uint4*>(xr + vi * 8);
      if (residual != nullptr) {
        Pack8 r;
        r.u = *reinterpret_cast<const uint4*>(residual + (size_t)row * H + vi * 8);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          // the sum is rounded to bf16 before it is normalised, as the stored residual is
          __nv_bfloat16 s = __float2bfloat16(__bfloat162float(a.h[j]) + __bfloat162float(r.h[j]));
          r.h[j] = s;
          v[i][j] = __bfloat162float(s);
        }
        *reinterpret_cast<uint4*>(residual + (size_t)row * H + vi * 8) = r.u;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] = __bfloat162float(a.h[j]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
    }
  }
  __shared__ float red[8];
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += red[i];
  const float rstd = rsqrtf(tot / (float)H + eps);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int vi = threadIdx.x + i * 256;
    if (vi < nvec) {
      Pack8 w, o;
      w.u = *reinterpret_cast<const uint4*>(weight + vi * 8);
      float y[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        o.h[j] = __float2bfloat16(v[i][j] * rstd * __bfloat162float(w.h[j]));
        y[j] = __bfloat162float(o.h[j]);
      }
      if (out != nullptr) *reinterpret_cast<uint4*>(out + (size_t)row * H + vi * 8) = o.u;
      if (out_q != nullptr) {
        // 16 consecutive threads hold one 128-wide quantisation block
        float m = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) m = fmaxf(m, fabsf(y[j]));
#pragma unroll
        for (int o2 = 8; o2 > 0; o2 >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o2));
        const float sc = fmaxf(m, 1e-10f) * (1.0f / 448.0f);
        const float inv = 1.0f / sc;
        uint8_t q[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) q[j] = f32_to_e4m3(y[j] * inv);
        *reinterpret_cast<uint2*>(out_q + (size_t)row * H + vi * 8) = *reinterpret_cast<uint2*>(q);
        if ((vi & 15) == 0) out_scale[(size_t)(vi >> 4) * out_scale_ld + row] = sc;
      }
    }
  }
}

// One warp per (row, 128-block) pair -> e4m3 + scale.
__global__ void quant_fp8_block_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* q, float* scale, int scale_ld,
                                       int T, int K, int x_ld, const int* __restrict__ row_limit) {
  const int nb = (K + 127) >> 7;
  const int wid = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= T * nb) return;
  const int row = wid / nb, b = wid - row * nb;
  if (row_limit != nullptr && row >= *row_limit) return;
  const int c = b * 128 + lane * 4;
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  if (c < K) {
    uint2 raw = *reinterpret_cast<const uint2*>(x + (size_t)row * x_ld + c);
    const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = (c + j < K) ? __bfloat162float(h[j]) : 0.f;
  }
  float m = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
  m = warp_max(m);
  const float sc = fmaxf(m, 1e-10f) * (1.0f / 448.0f);
  const float inv = 1.0f / sc;
  if (c < K) {
    uint8_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] = f32_to_e4m3(v[j] * inv);
    *reinterpret_cast<uint32_t*>(q + (size_t)row * K + c) = *reinterpret_cast<uint32_t*>(o);
  }
  if (lane == 0) scale[(size_t)b * scale_ld + row] = sc;
}

// MLA latent: one CTA (128 threads) per token.
//   latent [T, 576] bf16 = c_kv(512) | k_pe(64); cache row = slot * cache_ld.
//   cos_sin [max_pos, 64] fp32 = cos(32) | sin(32), already scaled by the YaRN mscale when one applies.
//   q (optional) [T, heads, q_ld_head] bf16: the last 64 values of every head are rotated in place.
__global__ void __launch_bounds__(128) mla_kv_rope_cache_kernel(
    const __nv_bfloat16* __restrict__ latent, int latent_ld, const __nv_bfloat16* __restrict__ kv_weight, float eps,
    const float* __restrict__ cos_sin, const int64_t* __restrict__ positions, const int64_t* __restrict__ slots,
    __nv_bfloat16* cache, int cache_ld, __nv_bfloat16* q, int heads, int q_head_dim, int q_rope_off,
    __nv_bfloat16* q_out, int q_out_head_dim, int q_out_off, __nv_bfloat16* latent_out) {
  const int t = blockIdx.x;
  const int64_t pos = positions[t];
  const int64_t slot = slots[t];
  const __nv_bfloat16* lr = latent + (size_t)t * latent_ld;
  const float* cs = cos_sin + (size_t)pos * 64;
  // --- RMSNorm over the 512 latent values: 128 threads x 4 values
  const int c = threadIdx.x * 4;
  uint2 raw = *reinterpret_cast<const uint2*>(lr + c);
  const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&raw);
  float v[4];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    v[j] = __bfloat162float(h[j]);
    ss += v[j] * v[j];
  }
  __shared__ float red[4];
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  const float rstd = rsqrtf((red[0] + red[1] + red[2] + red[3]) / 512.0f + eps);
  uint2 wraw = *reinterpret_cast<const uint2*>(kv_weight + c);
  const __nv_bfloat16* wh = reinterpret_cast<const __nv_bfloat16*>(&wraw);
  __nv_bfloat16 o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) o[j] = __float2bfloat16(v[j] * rstd * __bfloat162float(wh[j]));
  if (slot >= 0) *reinterpret_cast<uint2*>(cache + (size_t)slot * cache_ld + c) = *reinterpret_cast<uint2*>(o);
  if (latent_out) *reinterpret_cast<uint2*>(latent_out + (size_t)t * 576 + c) = *reinterpret_cast<uint2*>(o);
  // --- k_pe RoPE (interleaved pairs): threads 0..31 own one pair each
  if (threadIdx.x < 32) {
    const int i = threadIdx.x;
    const float cth = cs[i], sth = cs[32 + i];
    const float a = __bfloat162float(lr[512 + 2 * i]), b = __bfloat162float(lr[512 + 2 * i + 1]);
    __nv_bfloat162 r = __floats2bfloat162_rn(a * cth - b * sth, a * sth + b * cth);
    if (slot >= 0) *reinterpret_cast<__nv_bfloat162*>(cache + (size_t)slot * cache_ld + 512 + 2 * i) = r;
    if (latent_out) *reinterpret_cast<__nv_bfloat162*>(latent_out + (size_t)t * 576 + 512 + 2 * i) = r;
  }
  // --- q_pe RoPE for every head
  if (q != nullptr) {
    for (int idx = threadIdx.x; idx < heads * 32; idx += blockDim.x) {
      const int hd = idx >> 5, i = idx & 31;
      __nv_bfloat162* p2 =
          reinterpret_cast<__nv_bfloat162*>(q + ((size_t)t * heads + hd) * q_head_dim + q_rope_off + 2 * i);
      const float2 ab = __bfloat1622float2(*p2);
      const float cth = cs[i], sth = cs[32 + i];
      const __nv_bfloat162 rot = __floats2bfloat162_rn(ab.x * cth - ab.y * sth, ab.x * sth + ab.y * cth);
      if (q_out != nullptr)  // decode: rotated rope slice goes straight into the absorbed-q buffer
        *reinterpret_cast<__nv_bfloat162*>(q_out + ((size_t)t * heads + hd) * q_out_head_dim + q_out_off + 2 * i) = rot;
      else
        *p2 = rot;
    }
  }
}

// GQA: one CTA per token; one warp per head (q heads first, then k heads, then v heads).
//   qkv [T, (hq + 2*hkv) * D]; optional per-head RMSNorm weights (Qwen3); neox RoPE with cos_sin
//   [max_pos, D] = cos(D/2) | sin(D/2); k/v written to paged caches [slots, hkv*D] at slot.
__global__ void rope_qk_cache_kernel(__nv_bfloat16* qkv, int hq, int hkv, int D,
                                     const __nv_bfloat16* __restrict__ q_norm_w,
                                     const __nv_bfloat16* __restrict__ k_norm_w, float eps,
                                     const float* __restrict__ cos_sin, const int64_t* __restrict__ positions,
                                     const int64_t* __restrict__ slots, __nv_bfloat16* k_cache,
                                     __nv_bfloat16* v_cache) {
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nwarps = blockDim.x >> 5;
  const int64_t pos = positions[t];
  const int64_t slot = slots ? slots[t] : -1;
  const int half = D >> 1;
  const float* cs = cos_sin + (size_t)pos * D;
  __nv_bfloat16* row = qkv + (size_t)t * (hq + 2 * hkv) * D;
  for (int hd = warp; hd < hq + 2 * hkv; hd += nwarps) {
    __nv_bfloat16* p = row + (size_t)hd * D;
    if (hd >= hq + hkv) {  // v: plain copy into the cache
      if (slot >= 0)
        for (int i = lane; i < D; i += 32) v_cache[((size_t)slot * hkv + (hd - hq - hkv)) * D + i] = p[i];
      continue;
    }
    const __nv_bfloat16* nw = hd < hq ? q_norm_w : k_norm_w;
    float rstd = 1.f;
    if (nw != nullptr) {
      float ss = 0.f;
      for (int i = lane; i < D; i += 32) {
        float f = __bfloat162float(p[i]);
        ss += f * f;
      }
      rstd = rsqrtf(warp_sum(ss) / (float)D + eps);
    }
    for (int i = lane; i < half; i += 32) {
      float a = __bfloat162float(p[i]), b = __bfloat162float(p[i + half]);
      if (nw != nullptr) {
        a = __bfloat162float(__float2bfloat16(a * rstd * __bfloat162float(nw[i])));
        b = __bfloat162float(__float2bfloat16(b * rstd * __bfloat162float(nw[i + half])));
      }
      const float cth = cs[i], sth = cs[half + i];
      const __nv_bfloat16 ra = __float2bfloat16(a * cth - b * sth), rb = __float2bfloat16(b * cth + a * sth);
      p[i] = ra;
      p[i + half] = rb;
      if (hd >= hq && slot >= 0) {
        __nv_bfloat16* kc = k_cache + ((size_t)slot * hkv + (hd - hq)) * D;
        kc[i] = ra;
        kc[i + half] = rb;
      }
    }
  }
}

__global__ void silu_mul_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* out, int T, int I) {
  const size_t idx = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (idx >= (size_t)T * I) return;
  const size_t row = idx / I, c = idx - row * I;
  Pack8 g, u, o;
  g.u = *reinterpret_cast<const uint4*>(x + row * 2 * I + c);
  u.u = *reinterpret_cast<const uint4*>(x + row * 2 * I + I + c);
#pragma unroll
  for (int j = 0; j < 8; ++j) o.h[j] = __float2bfloat16(silu_f(__bfloat162float(g.h[j])) * __bfloat162float(u.h[j]));
  *reinterpret_cast<uint4*>(out + row * I + c) = o.u;
}

}  // namespace omni

using namespace omni;

extern "C" int omni_rmsnorm(const void* x, void* residual, const void* weight, void* out, void* out_q,
                            float* out_scale, int out_scale_ld, int T, int H, int x_ld, float eps,
                            cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H % 8 != 0 || H > 8 * 256 * 8) return -1;
  if (out_q != nullptr && H % 128 != 0) return -2;
  const int nvec = H / 8;
  const int vpt = (nvec + 255) / 256;
#define RMS_CASE(V)                                                                                              \
  if (vpt <= V) {                                                                                                \
    rmsnorm_kernel<V><<<T, 256, 0, stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)residual,                   \
                                             (const __nv_bfloat16*)weight, (__nv_bfloat16*)out, (uint8_t*)out_q, \
                                             out_scale, out_scale_ld, H, x_ld, eps);                             \
    return (int)cudaGetLastError();                                                                              \
  }
  RMS_CASE(1) RMS_CASE(2) RMS_CASE(4) RMS_CASE(8)
#undef RMS_CASE
  return -3;
}

extern "C" int omni_quant_fp8_block(const void* x, void* q, float* scale, int scale_ld, int T, int K, int x_ld,
                                    const int* row_limit, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (K % 4 != 0) return -1;
  const int nb = (K + 127) / 128;
  const long long warps = (long long)T * nb;
  const int blocks = (int)((warps * 32 + 255) / 256);
  quant_fp8_block_kernel<<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, (uint8_t*)q, scale, scale_ld, T, K,
                                                     x_ld, row_limit);
  return (int)cudaGetLastError();
}

extern "C" int omni_mla_kv_rope_cache(const void* latent, int latent_ld, const void* kv_weight, float eps,
                                      const float* cos_sin, const int64_t* positions, const int64_t* slots,
                                      void* cache, int cache_ld, void* q, int heads, int q_head_dim, int q_rope_off,
                                      void* q_out, int q_out_head_dim, int q_out_off, void* latent_out, int T,
                                      cudaStream_t stream) {
  if (T <= 0) return 0;
  mla_kv_rope_cache_kernel<<<T, 128, 0, stream>>>((const __nv_bfloat16*)latent, latent_ld,
                                                  (const __nv_bfloat16*)kv_weight, eps, cos_sin, positions, slots,
                                                  (__nv_bfloat16*)cache, cache_ld, (__nv_bfloat16*)q, heads,
                                                  q_head_dim, q_rope_off, (__nv_bfloat16*)q_out, q_out_head_dim,
                                                  q_out_off, (__nv_bfloat16*)latent_out);
  return (int)cudaGetLastError();
}

extern "C" int omni_rope_qk_cache(void* qkv, int hq, int hkv, int D, const void* q_norm_w, const void* k_norm_w,
                                  float eps, const float* cos_sin, const int64_t* positions, const int64_t* slots,
                                  void* k_cache, void* v_cache, int T, cudaStream_t stream) {
  if (T <= 0) return 0;
  rope_qk_cache_kernel<<<T, 256, 0, stream>>>((__nv_bfloat16*)qkv, hq, hkv, D, (const __nv_bfloat16*)q_norm_w,
                                              (const __nv_bfloat16*)k_norm_w, eps, cos_sin, positions, slots,
                                              (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache);
  return (int)cudaGetLastError();
}

extern "C" int omni_silu_mul(const void* x, void* out, int T, int I, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (I % 8 != 0) return -1;
  const size_t n = (size_t)T * I / 8;
  silu_mul_kernel<<<(int)((n + 255) / 256), 256, 0, stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)out, T, I);
  return (int)cudaGetLastError();
}
