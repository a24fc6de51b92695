// Small per-step device kernels that keep the decode loop free of host round trips:
//   omni_argmax           greedy token per row (bf16 or fp32 logits), optional (max,idx) pair output for
//                         vocab-parallel heads
//   omni_sample_topk_topp temperature / top-k / top-p sampling, one CTA per row (exact, sort-free:
//                         threshold search on the probability mass)
//   omni_apply_penalties  repetition / frequency / presence penalties from each row's token history
//   omni_mtp_verify       MTP draft verification and next drafter inputs
//   omni_step_advance     multi-step decode: positions+1, seq_lens+1, next slot from the block table
//   omni_embedding        (vocab-parallel) embedding gather
//   omni_omni_attn_slots  ring-window slot mapping of compressed Omni-Attention layers
// Reference behaviour: AscendSampler / SimpleSampler (omni/models/common/layers/sampler.py:331-511, 759-848),
// _simple_prepare_inputs (omni/adaptors/vllm/worker/npu_model_runner.py:347-407), VocabParallelEmbedding
// (omni/models/common/layers/vocab_parallel_embedding.py:140-165), compute_omni_attn_metadata
// (omni/accelerators/cache/utils.py:7-82).
#include "../include/omni_ptx.cuh"

namespace omni {

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__global__ void __launch_bounds__(1024) argmax_kernel(const T* __restrict__ logits, int V, int ld, int vocab_offset,
                                                      int64_t* out_ids, float* out_max) {
  const int row = blockIdx.x;
  const T* lr = logits + (size_t)row * ld;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = to_f<T>(lr[i]);
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  __shared__ float sv[32];
  __shared__ int si[32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { sv[warp] = best; si[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    best = lane < nw ? sv[lane] : -INFINITY;
    bi = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) {
      out_ids[row] = (int64_t)bi + vocab_offset;
      if (out_max) out_max[row] = best;
    }
  }
}

__device__ __forceinline__ float block_sum(float v, float* sbuf) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) sbuf[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) t += sbuf[i];
  return t;
}
__device__ __forceinline__ float block_max(float v, float* sbuf) {
  v = warp_max(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) sbuf[warp] = v;
  __syncthreads();
  float t = -INFINITY;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) t = fmaxf(t, sbuf[i]);
  return t;
}

// Sampling without a sort.  p_i = softmax(logit_i / temperature).  top-k and top-p both reduce to a
// probability threshold tau: keep {i : p_i >= tau}.  tau is found by bisection on [0, pmax] with block-wide
// count / mass reductions (24 rounds), then one inverse-CDF pass with the supplied uniform number picks the
// token among the kept ones in index order.
template <typename T>
__global__ void __launch_bounds__(1024) sample_kernel(const T* __restrict__ logits, int V, int ld,
                                                      const float* __restrict__ temperature,
                                                      const int* __restrict__ top_k, const float* __restrict__ top_p,
                                                      const float* __restrict__ uniform, int64_t* out_ids) {
  __shared__ float sbuf[32];
  __shared__ float scan[1024];
  const int row = blockIdx.x;
  const T* lr = logits + (size_t)row * ld;
  const float temp = temperature ? temperature[row] : 1.f;
  const int k = top_k ? top_k[row] : 0;
  const float pp = top_p ? top_p[row] : 1.f;
  if (temp < 1e-5f) {  // greedy row inside a sampling batch
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float v = to_f<T>(lr[i]);
      if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
    const float gmax = block_max(best, sbuf);
    int cand = (best == gmax) ? bi : 0x7fffffff;
    __shared__ int smin;
    if (threadIdx.x == 0) smin = 0x7fffffff;
    __syncthreads();
    atomicMin(&smin, cand);
    __syncthreads();
    if (threadIdx.x == 0) out_ids[row] = smin;
    return;
  }
  const float inv_t = 1.f / temp;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, to_f<T>(lr[i]) * inv_t);
  mx = block_max(mx, sbuf);
  float z = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) z += __expf(to_f<T>(lr[i]) * inv_t - mx);
  z = block_sum(z, sbuf);
  const float inv_z = 1.f / z;
  // threshold search
  float lo = 0.f, hi = inv_z;  // pmax = exp(0)/z
  const bool need = (k > 0 && k < V) || pp < 1.f;
  if (need) {
    for (int it = 0; it < 24; ++it) {
      const float mid = 0.5f * (lo + hi);
      float cnt = 0.f, mass = 0.f;
      for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float pr = __expf(to_f<T>(lr[i]) * inv_t - mx) * inv_z;
        if (pr >= mid) { cnt += 1.f; mass += pr; }
      }
      cnt = block_sum(cnt, sbuf);
      mass = block_sum(mass, sbuf);
      // {p >= mid} still satisfies a constraint (holds the k best, or holds mass >= pp): the
      // threshold may rise.  With both constraints active the kept set is the smaller of the two.
      const bool k_on = (k > 0 && k < V), p_on = (pp < 1.f);
      const bool can_raise = (k_on && cnt >= (float)k) || (p_on && mass >= pp);
      if (can_raise) lo = mid; else hi = mid;
    }
  }
  const float tau = need ? lo : 0.f;
  // kept mass
  float km = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float pr = __expf(to_f<T>(lr[i]) * inv_t - mx) * inv_z;
    if (pr >= tau) km += pr;
  }
  km = block_sum(km, sbuf);
  const float target = uniform[row] * km;
  // inverse CDF in index order: contiguous chunk per thread
  const int chunk = (V + blockDim.x - 1) / blockDim.x;
  const int b = threadIdx.x * chunk, e = min(V, b + chunk);
  float local = 0.f;
  for (int i = b; i < e; ++i) {
    const float pr = __expf(to_f<T>(lr[i]) * inv_t - mx) * inv_z;
    if (pr >= tau) local += pr;
  }
  scan[threadIdx.x] = local;
  __syncthreads();
  if (threadIdx.x == 0) {
    float acc = 0.f;
    int owner = -1;
    float before = 0.f;
    for (int i = 0; i < (int)blockDim.x; ++i) {
      if (scan[i] > 0.f) { owner = i; before = acc; }
      if (acc + scan[i] >= target && scan[i] > 0.f) { owner = i; before = acc; break; }
      acc += scan[i];
    }
    sbuf[0] = (float)owner;
    sbuf[1] = before;
  }
  __syncthreads();
  if ((int)sbuf[0] == (int)threadIdx.x) {
    float acc = sbuf[1];
    int pick = -1;
    for (int i = b; i < e; ++i) {
      const float pr = __expf(to_f<T>(lr[i]) * inv_t - mx) * inv_z;
      if (pr >= tau) {
        pick = i;
        acc += pr;
        if (acc >= target) break;
      }
    }
    out_ids[row] = pick;
  }
}

// input_ids / forward_tokens: [B, n] with n = 1 + num_speculative_tokens.
__global__ void mtp_verify_kernel(const int64_t* __restrict__ input_ids, const int64_t* __restrict__ forward_tokens,
                                  int B, int n, int64_t* out_tokens, int* accepted_num, int* last_accepted_index,
                                  int64_t* mtp_input_tokens, const float* __restrict__ accept_uniform,
                                  float control_accept_rate) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  int acc = n - 1;
  for (int i = 0; i < n - 1; ++i) {
    bool ok = input_ids[b * n + i + 1] == forward_tokens[b * n + i];
    if (accept_uniform != nullptr) ok = accept_uniform[b * (n - 1) + i] < control_accept_rate;
    if (!ok) { acc = i; break; }
  }
  accepted_num[b] = acc;
  last_accepted_index[b] = b * n + acc;
  for (int i = 0; i < n; ++i) {
    out_tokens[b * n + i] = (i <= acc) ? forward_tokens[b * n + i] : -1;
    mtp_input_tokens[b * n + i] = forward_tokens[b * n + i];
  }
}

// Multi-step decode: every live row advances by `advance[b]` (or 1) tokens.
__global__ void step_advance_kernel(int64_t* positions, int* seq_lens, int64_t* slots,
                                    const int* __restrict__ block_table, int bt_ld, int block_size, int B,
                                    int tokens_per_req, const int* __restrict__ advance) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const int adv = advance ? advance[b] : 1;
  if (seq_lens[b] <= 0) return;  // padding row
  const int new_len = seq_lens[b] + adv;
  seq_lens[b] = new_len;
  for (int j = 0; j < tokens_per_req; ++j) {
    const int64_t pos = (int64_t)new_len - tokens_per_req + j;
    positions[b * tokens_per_req + j] = pos;
    const int blk = block_table[(size_t)b * bt_ld + (int)(pos / block_size)];
    slots[b * tokens_per_req + j] = (int64_t)blk * block_size + (pos % block_size);
  }
}

__global__ void embedding_kernel(const int64_t* __restrict__ ids, const __nv_bfloat16* __restrict__ table, int H,
                                 int vocab_start, int vocab_end, __nv_bfloat16* out) {
  const int t = blockIdx.x;
  const int64_t id = ids[t];
  const bool mine = id >= vocab_start && id < vocab_end;
  const __nv_bfloat16* src = table + (size_t)(mine ? id - vocab_start : 0) * H;
  for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
    uint4 v = mine ? *reinterpret_cast<const uint4*>(src + c) : make_uint4(0, 0, 0, 0);
    *reinterpret_cast<uint4*>(out + (size_t)t * H + c) = v;
  }
}

// Compressed layers keep `sink` + `recent` blocks per request.  A token at sequence length L (1-based count
// after appending) goes to position L-1 while the request still fits, otherwise it wraps inside the recent
// window: window_pos = (L - base) % recent_tokens + sink_tokens, base = max(sink+recent tokens, prompt_len) + 1.
__global__ void omni_attn_slots_kernel(const int* __restrict__ seq_lens, const int* __restrict__ prompt_lens,
                                       const int* __restrict__ block_table, int bt_ld, int block_size, int sink,
                                       int recent, int B, int64_t* slots, int* eff_lens) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const int L = seq_lens[b];
  if (L <= 0) { slots[b] = -1; if (eff_lens) eff_lens[b] = 0; return; }
  const int sink_tokens = sink * block_size, recent_tokens = recent * block_size;
  const int cap = sink_tokens + recent_tokens;
  int pos;
  if (L <= cap) pos = L - 1;
  else {
    const int base = max(cap, prompt_lens[b]) + 1;
    int m = (L - base) % recent_tokens;
    if (m < 0) m += recent_tokens;
    pos = m + sink_tokens;
  }
  const int blk = block_table[(size_t)b * bt_ld + pos / block_size];
  slots[b] = (int64_t)blk * block_size + pos % block_size;
  if (eff_lens) eff_lens[b] = min(L, cap);
}


// Sampling penalties, one CTA per row (omni/models/common/layers/sampler.py:143-200).  hist[row, :] holds the
// row's prompt tokens followed by its output tokens, -1 padded; the first prompt_len[row] entries are prompt.
//   repetition: logits of tokens seen in prompt or output are divided (if > 0) or multiplied (if <= 0) by rep
//   frequency:  logits -= freq * (occurrences among the output tokens)
//   presence:   logits -= pres * (token occurs among the output tokens)
// counts[row, :] (int32 per vocabulary entry) is scratch owned by the row's CTA: cleared, filled with atomics
// (bit 30 = "seen in the prompt", low bits = output occurrences), then read back.  Rows whose three
// parameters are neutral return at once.
template <typename T>
__global__ void __launch_bounds__(1024) penalties_kernel(T* __restrict__ logits, int V, int ld, const int* __restrict__ hist,
                                                        int hist_ld, const int* __restrict__ prompt_len,
                                                        const float* __restrict__ rep, const float* __restrict__ freq,
                                                        const float* __restrict__ pres, int* __restrict__ counts) {
  const int row = blockIdx.x;
  const float r = rep[row], f = freq[row], pz = pres[row];
  if (r == 1.0f && f == 0.0f && pz == 0.0f) return;
  int* cnt = counts + (size_t)row * V;
  for (int i = threadIdx.x; i < V; i += blockDim.x) cnt[i] = 0;
  __syncthreads();
  const int* h = hist + (size_t)row * hist_ld;
  const int np = prompt_len[row];
  for (int i = threadIdx.x; i < hist_ld; i += blockDim.x) {
    const int t = h[i];
    if (t < 0 || t >= V) continue;
    if (i < np) atomicOr(&cnt[t], 1 << 30);
    else atomicAdd(&cnt[t], 1);
  }
  __syncthreads();
  T* lr = logits + (size_t)row * ld;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const int c = cnt[i];
    if (c == 0) continue;
    float v = to_f<T>(lr[i]);
    if (r != 1.0f) v = v > 0.f ? v / r : v * r;
    const int n_out = c & ((1 << 30) - 1);
    if (n_out > 0) v -= f * (float)n_out + pz;
    lr[i] = (T)v;
  }
}

}  // namespace omni

using namespace omni;

extern "C" int omni_argmax(const void* logits, int is_bf16, int B, int V, int ld, int vocab_offset, int64_t* out_ids,
                           float* out_max, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (is_bf16)
    argmax_kernel<__nv_bfloat16><<<B, 1024, 0, stream>>>((const __nv_bfloat16*)logits, V, ld, vocab_offset, out_ids,
                                                         out_max);
  else
    argmax_kernel<float><<<B, 1024, 0, stream>>>((const float*)logits, V, ld, vocab_offset, out_ids, out_max);
  return (int)cudaGetLastError();
}

extern "C" int omni_sample_topk_topp(const void* logits, int is_bf16, int B, int V, int ld, const float* temperature,
                                     const int* top_k, const float* top_p, const float* uniform, int64_t* out_ids,
                                     cudaStream_t stream) {
  if (B <= 0) return 0;
  if (is_bf16)
    sample_kernel<__nv_bfloat16><<<B, 1024, 0, stream>>>((const __nv_bfloat16*)logits, V, ld, temperature, top_k,
                                                         top_p, uniform, out_ids);
  else
    sample_kernel<float><<<B, 1024, 0, stream>>>((const float*)logits, V, ld, temperature, top_k, top_p, uniform,
                                                 out_ids);
  return (int)cudaGetLastError();
}

extern "C" int omni_mtp_verify(const int64_t* input_ids, const int64_t* forward_tokens, int B, int n,
                               int64_t* out_tokens, int* accepted_num, int* last_accepted_index,
                               int64_t* mtp_input_tokens, const float* accept_uniform, float control_accept_rate,
                               cudaStream_t stream) {
  if (B <= 0) return 0;
  mtp_verify_kernel<<<(B + 127) / 128, 128, 0, stream>>>(input_ids, forward_tokens, B, n, out_tokens, accepted_num,
                                                         last_accepted_index, mtp_input_tokens, accept_uniform,
                                                         control_accept_rate);
  return (int)cudaGetLastError();
}

extern "C" int omni_step_advance(int64_t* positions, int* seq_lens, int64_t* slots, const int* block_table, int bt_ld,
                                 int block_size, int B, int tokens_per_req, const int* advance,
                                 cudaStream_t stream) {
  if (B <= 0) return 0;
  step_advance_kernel<<<(B + 127) / 128, 128, 0, stream>>>(positions, seq_lens, slots, block_table, bt_ld, block_size,
                                                           B, tokens_per_req, advance);
  return (int)cudaGetLastError();
}

extern "C" int omni_embedding(const int64_t* ids, const void* table, int T, int H, int vocab_start, int vocab_end,
                              void* out, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H % 8 != 0) return -1;
  int threads = H / 8;
  if (threads > 256) threads = 256;
  embedding_kernel<<<T, threads, 0, stream>>>(ids, (const __nv_bfloat16*)table, H, vocab_start, vocab_end,
                                              (__nv_bfloat16*)out);
  return (int)cudaGetLastError();
}

extern "C" int omni_omni_attn_slots(const int* seq_lens, const int* prompt_lens, const int* block_table, int bt_ld,
                                    int block_size, int sink, int recent, int B, int64_t* slots, int* eff_lens,
                                    cudaStream_t stream) {
  if (B <= 0) return 0;
  omni_attn_slots_kernel<<<(B + 127) / 128, 128, 0, stream>>>(seq_lens, prompt_lens, block_table, bt_ld, block_size,
                                                              sink, recent, B, slots, eff_lens);
  return (int)cudaGetLastError();
}

// In place on logits [B, V] (fp32 or bf16).  counts: int32 scratch [B, V].
extern "C" int omni_apply_penalties(void* logits, int is_bf16, int B, int V, int ld, const int* hist, int hist_ld,
                                    const int* prompt_len, const float* rep, const float* freq, const float* pres,
                                    int* counts, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (hist == nullptr || counts == nullptr) return -1;
  if (is_bf16)
    penalties_kernel<__nv_bfloat16><<<B, 1024, 0, stream>>>((__nv_bfloat16*)logits, V, ld, hist, hist_ld, prompt_len, rep,
                                                            freq, pres, counts);
  else
    penalties_kernel<float><<<B, 1024, 0, stream>>>((float*)logits, V, ld, hist, hist_ld, prompt_len, rep, freq, pres, counts);
  return (int)cudaGetLastError();
}
