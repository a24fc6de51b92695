// MoE routing and local (single-rank) token permutation.
//   omni_router_topk   scores (softmax | sigmoid + selection bias), group-limited top-k, renormalise,
//                      routed scaling, logical->physical remap through a selector table, activation
//                      histogram.  One warp per token.
//   omni_moe_align     per-expert counts, 16-row aligned segment starts, slot of every (token, k)
//   omni_moe_scatter   gather token rows into expert-sorted order (bf16 copy or e4m3 1x128 quantisation)
//   omni_moe_combine   out[t] = sum_k y[row_of[t,k]] (+ shared-expert output)
// Semantics follow the reference's grouped_topk / fused_topk / npu_moe_gating_top_k call sites
// (omni/models/common/layers/moe/fused_moe/fused_moe.py:24-84, .../fused_moe/layer.py:302-365), the
// planner remap (omni/accelerators/placement/omni_planner/omni_planner.py:244-274) and the
// init_routing / finalize_routing pair (fused_moe.py:109-186).
#include "../include/omni_ptx.cuh"

namespace omni {

constexpr int ROUTER_MAX_PER_LANE = 16;  // experts <= 512

struct RouterParams {
  const float* logits;    // [T, E]
  const float* bias;      // [E] or null (added for selection only)
  int T, E;
  int mode;               // 0 softmax, 1 sigmoid
  int n_group, topk_group;
  int group_mode;         // 0: group score = max, 1: sum of the two best
  int top_k;
  int renorm;
  float scale;
  const int* selector;    // [E] logical -> physical, or null
  unsigned long long* counts;  // [n_counts] activation histogram over physical positions, or null
  int n_counts;
  OmniStatus* st;         // a row without any selectable expert (all scores NaN) or a selector entry outside the
                          // histogram is reported here and the pair is dropped (id -1, weight 0)
  int forced_balance;     // ids = round robin (benchmark aid), weights uniform
  const int* num_valid;   // optional device scalar: rows >= *num_valid are padding
  int* out_ids;           // [T, top_k]
  float* out_w;           // [T, top_k]
};

__global__ void __launch_bounds__(128) router_topk_kernel(const RouterParams p) {
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= p.T) return;
  const bool padded = p.num_valid != nullptr && t >= *p.num_valid;
  float* sel = sm + (size_t)warp * p.E;  // selection scores of this token
  const int per_lane = (p.E + 31) >> 5;
  float score[ROUTER_MAX_PER_LANE];
  const float* lg = p.logits + (size_t)t * p.E;

  if (p.forced_balance || padded) {
    for (int j = lane; j < p.top_k; j += 32) {
      int id = (int)(((long long)t * p.top_k + j) % p.E);
      if (p.selector) id = p.selector[id];
      p.out_ids[(size_t)t * p.top_k + j] = padded ? -1 : id;
      p.out_w[(size_t)t * p.top_k + j] = padded ? 0.f : p.scale / (float)p.top_k;
      if (p.counts && !padded && id >= 0 && id < p.n_counts) atomicAdd(&p.counts[id], 1ull);
    }
    return;
  }

  // ---- scores
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < ROUTER_MAX_PER_LANE; ++i) {
    const int e = i * 32 + lane;
    score[i] = (i < per_lane && e < p.E) ? lg[e] : -INFINITY;
    mx = fmaxf(mx, score[i]);
  }
  if (p.mode == 0) {
    mx = warp_max(mx);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < ROUTER_MAX_PER_LANE; ++i) {
      const int e = i * 32 + lane;
      score[i] = (i < per_lane && e < p.E) ? __expf(score[i] - mx) : 0.f;
      s += score[i];
    }
    s = warp_sum(s);
    const float inv = 1.f / s;
#pragma unroll
    for (int i = 0; i < ROUTER_MAX_PER_LANE; ++i) score[i] *= inv;
  } else {
#pragma unroll
    for (int i = 0; i < ROUTER_MAX_PER_LANE; ++i) score[i] = 1.f / (1.f + __expf(-score[i]));
  }
  // selection score (biased) into shared memory
#pragma unroll
  for (int i = 0; i < ROUTER_MAX_PER_LANE; ++i) {
    const int e = i * 32 + lane;
    if (i < per_lane && e < p.E) sel[e] = score[i] + (p.bias ? p.bias[e] : 0.f);
  }
  __syncwarp();

  // ---- group-limited routing: keep the best `topk_group` groups
  if (p.n_group > 1) {
    const int gs = p.E / p.n_group;
    float gscore = -INFINITY;
    if (lane < p.n_group) {
      float b1 = -INFINITY, b2 = -INFINITY;
      for (int j = 0; j < gs; ++j) {
        const float v = sel[lane * gs + j];
        if (v > b1) { b2 = b1; b1 = v; } else if (v > b2) { b2 = v; }
      }
      gscore = p.group_mode == 1 ? b1 + b2 : b1;
    }
    unsigned keep = 0;
    for (int r = 0; r < p.topk_group; ++r) {
      float v = gscore;
      int idx = lane;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
      }
      keep |= 1u << idx;
      if (lane == idx) gscore = -INFINITY;
    }
    for (int e = lane; e < p.E; e += 32)
      if (!((keep >> (e / gs)) & 1u)) sel[e] = -INFINITY;
    __syncwarp();
  }

  // ---- top-k by repeated warp arg-max over the selection scores
  float wsum = 0.f;
  float my_w = 0.f;
  int my_id = -1;
  for (int r = 0; r < p.top_k; ++r) {
    float v = -INFINITY;
    int idx = 0x7fffffff;
    for (int e = lane; e < p.E; e += 32) {
      const float s = sel[e];
      if (s > v) { v = s; idx = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
      if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
    // un-biased score of the winner lives in lane (idx & 31), register (idx >> 5)
    float w = 0.f;
#pragma unroll
    for (int i = 0; i < ROUTER_MAX_PER_LANE; ++i)
      if (i == (idx >> 5)) w = score[i];
    w = __shfl_sync(0xffffffffu, w, idx & 31);
    wsum += w;
    if (lane == r) { my_w = w; my_id = idx; }
    if (idx < p.E && lane == (idx & 31)) sel[idx] = -INFINITY;
    __syncwarp();
  }
  if (lane < p.top_k) {
    float w = my_w;
    if (p.renorm) w = w / (wsum + 1e-20f);
    w *= p.scale;
    int id = my_id;
    if (id < 0 || id >= p.E) {                 // nothing compared greater than -inf: the scores of this row are NaN
      report_status(p.st, OMNI_ERR_BOUNDS, 1, t);
      id = -1;
      w = 0.f;
    } else if (p.selector) {
      id = p.selector[id];
    }
    if (p.counts && id >= 0) {
      if (id < p.n_counts) {
        atomicAdd(&p.counts[id], 1ull);
      } else {
        report_status(p.st, OMNI_ERR_BOUNDS, 2, id);
        id = -1;
        w = 0.f;
      }
    }
    p.out_ids[(size_t)t * p.top_k + lane] = id;
    p.out_w[(size_t)t * p.top_k + lane] = w;
  }
}

// ---- local permutation -----------------------------------------------------------------------
// counts[e] (zeroed by the caller) -> slot of each (t,k) inside its expert
__global__ void moe_count_kernel(const int* __restrict__ ids, int n, int e_lo, int e_local, int* counts, int* pos) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int e = ids[i] - e_lo;
  pos[i] = (e >= 0 && e < e_local) ? atomicAdd(&counts[e], 1) : -1;
}

// single CTA: aligned exclusive prefix
__global__ void moe_prefix_kernel(const int* __restrict__ counts, int e_local, int align, int* seg_start,
                                  int* seg_len, int* total_rows, int capacity, OmniStatus* status) {
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < e_local; ++e) {
      seg_start[e] = acc;
      int c = counts[e];
      if (acc + c > capacity) {  // never write past the permuted buffer: clip and report
        report_status(status, OMNI_ERR_CAPACITY, 100, e);
        c = max(0, capacity - acc);
      }
      seg_len[e] = c;
      acc += (c + align - 1) / align * align;
    }
    *total_rows = acc;
  }
}

// one warp per (t,k): copy / quantise the token row into its expert-sorted slot
__global__ void moe_scatter_kernel(const __nv_bfloat16* __restrict__ x, int H, const int* __restrict__ ids,
                                   const float* __restrict__ w, const int* __restrict__ pos, int n, int top_k,
                                   int e_lo, const int* __restrict__ seg_start, const int* __restrict__ seg_len,
                                   __nv_bfloat16* xp, uint8_t* xq, float* xs, int xs_ld, int* row_of,
                                   float* row_w, int* src_of) {
  const int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (i >= n) return;
  const int ps = pos[i];
  const int e = ids[i] - e_lo;
  if (ps < 0 || ps >= seg_len[e]) {
    if (lane == 0) row_of[i] = -1;
    return;
  }
  const int row = seg_start[e] + ps;
  const int t = i / top_k;
  if (lane == 0) {
    row_of[i] = row;
    row_w[row] = w[i];
    if (src_of) src_of[row] = i;
  }
  const __nv_bfloat16* src = x + (size_t)t * H;
  if (xq == nullptr) {
    for (int c = lane * 8; c < H; c += 256)
      *reinterpret_cast<uint4*>(xp + (size_t)row * H + c) = *reinterpret_cast<const uint4*>(src + c);
  } else {
    // each warp iteration covers one 128-wide block: 4 values per lane
    for (int b = 0; b < (H >> 7); ++b) {
      const int c = b * 128 + lane * 4;
      uint2 raw = *reinterpret_cast<const uint2*>(src + c);
      const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&raw);
      float v[4];
      float m = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[j] = __bfloat162float(h[j]);
        m = fmaxf(m, fabsf(v[j]));
      }
      m = warp_max(m);
      const float sc = fmaxf(m, 1e-10f) * (1.0f / 448.0f);
      const float inv = 1.0f / sc;
      uint8_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = f32_to_e4m3(v[j] * inv);
      *reinterpret_cast<uint32_t*>(xq + (size_t)row * H + c) = *reinterpret_cast<uint32_t*>(o);
      if (lane == 0) xs[(size_t)b * xs_ld + row] = sc;
    }
  }
}

// same for rows that are already quantised (the e4m3 output of the preceding RMSNorm): a token routed to k local
// experts is copied k times instead of being quantised k times.  xs_in is K-block major [H/128, xs_in_ld].
__global__ void moe_scatter_q8_kernel(const uint8_t* __restrict__ xq_in, const float* __restrict__ xs_in, int xs_in_ld, int H,
                                      const int* __restrict__ ids, const float* __restrict__ w, const int* __restrict__ pos,
                                      int n, int top_k, int e_lo, const int* __restrict__ seg_start,
                                      const int* __restrict__ seg_len, uint8_t* xq, float* xs, int xs_ld, int* row_of,
                                      float* row_w, int* src_of) {
  const int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (i >= n) return;
  const int ps = pos[i];
  const int e = ids[i] - e_lo;
  if (ps < 0 || ps >= seg_len[e]) {
    if (lane == 0) row_of[i] = -1;
    return;
  }
  const int row = seg_start[e] + ps;
  const int t = i / top_k;
  if (lane == 0) {
    row_of[i] = row;
    row_w[row] = w[i];
    if (src_of) src_of[row] = i;
  }
  const uint4* src = reinterpret_cast<const uint4*>(xq_in + (size_t)t * H);
  uint4* dst = reinterpret_cast<uint4*>(xq + (size_t)row * H);
  for (int c = lane; c < (H >> 4); c += 32) dst[c] = __ldg(src + c);
  for (int b = lane; b < (H >> 7); b += 32) xs[(size_t)b * xs_ld + row] = __ldg(xs_in + (size_t)b * xs_in_ld + t);
}

// one CTA per token: fixed summation order over k (deterministic)
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ y, int H, const int* __restrict__ row_of,
                                   const float* __restrict__ w, int top_k, const __nv_bfloat16* __restrict__ shared,
                                   __nv_bfloat16* out) {
  // gridDim.y column parts per token: a decode batch has only a few hundred tokens, one CTA each would leave SMs idle
  const int t = blockIdx.x;
  const int part = (H / 8 + gridDim.y - 1) / gridDim.y * 8;
  const int c_lo = blockIdx.y * part, c_hi = min(H, c_lo + part);
  for (int c = c_lo + threadIdx.x * 8; c < c_hi; c += blockDim.x * 8) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll 4
    for (int k = 0; k < top_k; ++k) {
      const int row = row_of[t * top_k + k];
      if (row < 0) continue;
      const float wk = w ? w[t * top_k + k] : 1.f;
      uint4 raw = *reinterpret_cast<const uint4*>(y + (size_t)row * H + c);
      const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += wk * __bfloat162float(h[j]);
    }
    if (shared) {
      uint4 raw = *reinterpret_cast<const uint4*>(shared + (size_t)t * H + c);
      const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += __bfloat162float(h[j]);
    }
    __nv_bfloat16 o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = __float2bfloat16(acc[j]);
    *reinterpret_cast<uint4*>(out + (size_t)t * H + c) = *reinterpret_cast<uint4*>(o);
  }
}

}  // namespace omni

using namespace omni;

extern "C" int omni_router_topk(const float* logits, const float* bias, int T, int E, int mode, int n_group,
                                int topk_group, int group_mode, int top_k, int renorm, float scale,
                                const int* selector, void* counts, int n_counts, int forced_balance,
                                const int* num_valid, int* out_ids, float* out_w, void* status,
                                cudaStream_t stream) {
  if (T <= 0) return 0;
  if (E > 32 * ROUTER_MAX_PER_LANE || top_k > 32 || top_k > E) return -1;
  if (n_group > 32 || (n_group > 1 && E % n_group != 0)) return -2;
  RouterParams p;
  p.logits = logits; p.bias = bias; p.T = T; p.E = E; p.mode = mode; p.n_group = n_group;
  p.topk_group = topk_group; p.group_mode = group_mode; p.top_k = top_k; p.renorm = renorm; p.scale = scale;
  p.selector = selector; p.counts = (unsigned long long*)counts; p.forced_balance = forced_balance;
  p.n_counts = n_counts; p.st = (OmniStatus*)status;
  p.num_valid = num_valid; p.out_ids = out_ids; p.out_w = out_w;
  const int warps = 4;
  router_topk_kernel<<<(T + warps - 1) / warps, warps * 32, warps * E * sizeof(float), stream>>>(p);
  return (int)cudaGetLastError();
}

// counts must hold e_local ints; it is cleared here.
extern "C" int omni_moe_align(const int* ids, int n, int e_lo, int e_local, int align, int capacity, int* counts,
                              int* pos, int* seg_start, int* seg_len, int* total_rows, void* status,
                              cudaStream_t stream) {
  cudaMemsetAsync(counts, 0, sizeof(int) * e_local, stream);
  if (n > 0) moe_count_kernel<<<(n + 255) / 256, 256, 0, stream>>>(ids, n, e_lo, e_local, counts, pos);
  moe_prefix_kernel<<<1, 32, 0, stream>>>(counts, e_local, align, seg_start, seg_len, total_rows, capacity,
                                          (OmniStatus*)status);
  return (int)cudaGetLastError();
}

extern "C" int omni_moe_scatter(const void* x, int H, const int* ids, const float* w, const int* pos, int n,
                                int top_k, int e_lo, const int* seg_start, const int* seg_len, void* xp, void* xq,
                                float* xs, int xs_ld, int* row_of, float* row_w, int* src_of,
                                cudaStream_t stream) {
  if (n <= 0) return 0;
  if (H % 8 != 0 || (xq != nullptr && H % 128 != 0)) return -1;
  const long long threads = (long long)n * 32;
  moe_scatter_kernel<<<(int)((threads + 255) / 256), 256, 0, stream>>>(
      (const __nv_bfloat16*)x, H, ids, w, pos, n, top_k, e_lo, seg_start, seg_len, (__nv_bfloat16*)xp, (uint8_t*)xq,
      xs, xs_ld, row_of, row_w, src_of);
  return (int)cudaGetLastError();
}

extern "C" int omni_moe_scatter_q8(const void* xq_in, const float* xs_in, int xs_in_ld, int H, const int* ids, const float* w,
                                   const int* pos, int n, int top_k, int e_lo, const int* seg_start, const int* seg_len,
                                   void* xq, float* xs, int xs_ld, int* row_of, float* row_w, int* src_of,
                                   cudaStream_t stream) {
  if (n <= 0) return 0;
  if (H % 128 != 0 || xq_in == nullptr || xs_in == nullptr || xq == nullptr || xs == nullptr) return -1;
  const long long threads = (long long)n * 32;
  moe_scatter_q8_kernel<<<(int)((threads + 255) / 256), 256, 0, stream>>>(
      (const uint8_t*)xq_in, xs_in, xs_in_ld, H, ids, w, pos, n, top_k, e_lo, seg_start, seg_len, (uint8_t*)xq, xs, xs_ld,
      row_of, row_w, src_of);
  return (int)cudaGetLastError();
}

extern "C" int omni_moe_combine(const void* y, int H, const int* row_of, const float* w, int T, int top_k,
                                const void* shared, void* out, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H % 8 != 0) return -1;
  int parts = 1;
  while (T * parts < 1184 && parts < 8 && H / (parts * 2) >= 512) parts *= 2;   // aim at 8 CTAs per SM
  int threads = (H / parts + 7) / 8;
  threads = (threads + 31) / 32 * 32;
  if (threads > 256) threads = 256;
  moe_combine_kernel<<<dim3(T, parts), threads, 0, stream>>>((const __nv_bfloat16*)y, H, row_of, w, top_k,
                                                (const __nv_bfloat16*)shared, (__nv_bfloat16*)out);
  return (int)cudaGetLastError();
}
