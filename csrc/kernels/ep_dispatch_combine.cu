// Expert-parallel dispatch and combine over NVLink peer memory (no NCCL on this path).
//
// Every rank owns one "symmetric" buffer allocated with cudaMalloc and opened by all peers through CUDA IPC;
// `peer[r]` is rank r's buffer as seen from this rank, the layout (EpLayout) is identical on all ranks.
//
//   dispatch  omni_ep_dispatch_send   one warp per (token, k): quantises the token row to e4m3 with 1x128 scales (or
//                                     copies the e4m3 form the caller already has, or the bf16 row for models with
//                                     unquantised experts) and stores row + scales + {local expert, source slot, weight} straight into
//                                     the destination rank's receive region over NVLink; the last block publishes
//                                     per-destination counts and release-stores one flag per destination
//             omni_ep_dispatch_recv   bounded wait on the flags of all sources, then compacts the received
//                                     metadata into a dense id list (the local permutation kernels sort it)
//             omni_ep_scatter_q       copies received rows into expert-sorted order (scales transposed to the
//                                     K-block-major layout the grouped GEMM reads)
//   combine   omni_ep_combine_send    returns expert outputs to the rank and (token, k) slot they came from
//             omni_ep_combine_reduce  bounded wait on all ranks, then out[t] = sum_k slot[t,k] (+ shared expert),
//                                     fixed order over k
//
// Flags carry an epoch that each rank keeps in its own buffer and advances inside the kernels, so the same
// launches can be replayed from a CUDA graph.  A wait that runs out records a status word and the kernel goes on
// with what it has (outputs of missing peers are zero); nothing traps or spins forever.
// Buffer reuse is safe without extra barriers: a rank starts the next dispatch only after its combine_reduce saw
// every peer's flag, and a peer sends combine data only after it has finished reading its receive region.
//
// These kernels take the place of the reference's npu_moe_distribute_dispatch / npu_moe_distribute_combine
// (omni/models/common/layers/moe/deepseek_moe.py:407-439, 495-536).
#include <string.h>

#include "../include/omni_ptx.cuh"

namespace omni {

struct EpLayout {
  int world, rank;
  int cap;              // receive rows reserved per source rank
  int H;                // hidden size (multiple of 128)
  int max_slots;        // T_max * top_k rows of the combine buffer
  int payload;          // dispatched rows: 1 (or 0) = e4m3 with 1x128 scales, 2 = bf16 without scales
  // byte offsets inside the symmetric buffer
  long long off_recv_x, off_recv_s, off_recv_meta, off_recv_cnt, off_recv_flag, off_comb, off_comb_flag, off_ctrl;
};
// ctrl (local only): [0] dispatch epoch, [1] combine epoch, [2] done-blocks (dispatch), [3] done-blocks (combine),
//                    [8 .. 8+world) send counts per destination
struct EpMeta { int expert; int slot; float weight; int pad; };

struct EpPeers { unsigned char* p[16]; };

__device__ __forceinline__ void st_v4_u32(void* p, uint4 v) { *reinterpret_cast<uint4*>(p) = v; }

__global__ void __launch_bounds__(256)
ep_dispatch_send_kernel(const __nv_bfloat16* __restrict__ x, const uint8_t* __restrict__ xq_in,
                        const float* __restrict__ xs_in, int xs_in_ld, const int* __restrict__ ids,
                        const float* __restrict__ w, int n_pairs, int top_k, int slots_per_rank, EpLayout L,
                        EpPeers peers, OmniStatus* status) {
  unsigned char* self = peers.p[L.rank];
  int* ctrl = reinterpret_cast<int*>(self + L.off_ctrl);
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int H = L.H, nb = H >> 7;
  for (int i = blockIdx.x * warps_per_block + (threadIdx.x >> 5); i < n_pairs; i += gridDim.x * warps_per_block) {
    const int id = ids[i];
    if (id < 0) continue;                      // padding row
    const int d = id / slots_per_rank, e = id - d * slots_per_rank;
    int slot = 0;
    if (lane == 0) slot = atomicAdd(&ctrl[8 + d], 1);
    slot = __shfl_sync(0xffffffffu, slot, 0);
    if (slot >= L.cap) {                       // never write past the region: drop and report
      if (lane == 0) report_status(status, OMNI_ERR_CAPACITY, 200, d);
      // nobody will answer for this pair, and its row of the combine buffer still holds an older round's output for
      // some other token: clear it, so that the reduction adds zero (the previous round's reduction has finished:
      // it ran earlier on this stream)
      uint4* z4 = reinterpret_cast<uint4*>(self + L.off_comb + (size_t)i * H * 2);
      for (int c = lane; c < (H >> 3); c += 32) z4[c] = make_uint4(0u, 0u, 0u, 0u);
      continue;
    }
    unsigned char* dst = peers.p[d];
    const size_t rrow = (size_t)L.rank * L.cap + slot;
    const int t = i / top_k;
    if (L.payload == 2) {
      // bf16 rows travel as they are (models whose experts are not quantised)
      const uint4* s4 = reinterpret_cast<const uint4*>(x + (size_t)t * H);
      uint4* d4 = reinterpret_cast<uint4*>(dst + L.off_recv_x + rrow * (size_t)H * 2);
      for (int c = lane; c < (H >> 3); c += 32) d4[c] = __ldg(s4 + c);
    } else if (xq_in != nullptr) {
      // the caller already has the e4m3 form of the rows (output of the preceding RMSNorm): copy, do not re-quantise
      const uint4* s4 = reinterpret_cast<const uint4*>(xq_in + (size_t)t * H);
      uint4* d4 = reinterpret_cast<uint4*>(dst + L.off_recv_x + rrow * H);
      for (int c = lane; c < (H >> 4); c += 32) d4[c] = __ldg(s4 + c);
      float* xs = reinterpret_cast<float*>(dst + L.off_recv_s) + rrow * nb;
      for (int b = lane; b < nb; b += 32) xs[b] = __ldg(xs_in + (size_t)b * xs_in_ld + t);
    } else {
    uint8_t* xq = dst + L.off_recv_x + rrow * H;
    float* xs = reinterpret_cast<float*>(dst + L.off_recv_s) + rrow * nb;
    const __nv_bfloat16* src = x + (size_t)t * H;
    for (int b = 0; b < nb; ++b) {
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
      *reinterpret_cast<uint32_t*>(xq + c) = *reinterpret_cast<uint32_t*>(o);   // 128 B per warp store
      if (lane == 0) xs[b] = sc;
    }
    }
    if (lane == 0) {
      EpMeta mt;
      mt.expert = e; mt.slot = i; mt.weight = w[i]; mt.pad = 0;
      *reinterpret_cast<EpMeta*>(dst + L.off_recv_meta + rrow * sizeof(EpMeta)) = mt;
    }
  }
  // ---- completion: the last block publishes counts, then flags (release at system scope)
  __threadfence_system();
  __syncthreads();
  __shared__ int is_last;
  if (threadIdx.x == 0) is_last = (atomicAdd(&ctrl[2], 1) == (int)gridDim.x - 1);
  __syncthreads();
  if (is_last) {
    __threadfence_system();
    const int epoch = ctrl[0] + 1;
    if ((int)threadIdx.x < L.world) {
      const int d = threadIdx.x;
      int* cnt = reinterpret_cast<int*>(peers.p[d] + L.off_recv_cnt);
      int* flag = reinterpret_cast<int*>(peers.p[d] + L.off_recv_flag);
      cnt[L.rank] = min(ctrl[8 + d], L.cap);
      __threadfence_system();
      st_release_sys(&flag[L.rank], epoch);
      ctrl[8 + d] = 0;
    }
    __syncthreads();
    if (threadIdx.x == 0) { ctrl[0] = epoch; ctrl[2] = 0; }
  }
}

// Waits for every source, then writes ids_out[src*cap + j] = local expert (or -1), w_out, slot_out.
__global__ void __launch_bounds__(1024)
ep_dispatch_recv_kernel(EpLayout L, EpPeers peers, int* ids_out, float* w_out, int* src_slot_out, int* counts_out,
                        unsigned long long wait_ns, OmniStatus* status) {
  unsigned char* self = peers.p[L.rank];
  int* ctrl = reinterpret_cast<int*>(self + L.off_ctrl);
  const int* cnt = reinterpret_cast<const int*>(self + L.off_recv_cnt);
  const int* flag = reinterpret_cast<const int*>(self + L.off_recv_flag);
  __shared__ int n_from[16];
  // the send kernel of this rank ran first on the same stream, so ctrl[0] already holds this round's epoch
  const int epoch = ctrl[0];
  if ((int)threadIdx.x < L.world) {
    const bool ok = flag_wait_ge(&flag[threadIdx.x], epoch, wait_ns, status, 201, threadIdx.x);
    n_from[threadIdx.x] = ok ? ld_relaxed_sys(&cnt[threadIdx.x]) : 0;
    if (counts_out && blockIdx.x == 0) counts_out[threadIdx.x] = n_from[threadIdx.x];
  }
  __syncthreads();
  // every block waits for the flags itself (they are already set for all but the first to arrive), then takes its
  // share of the world * cap metadata slots
  const EpMeta* meta = reinterpret_cast<const EpMeta*>(self + L.off_recv_meta);
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < L.world * L.cap; i += gridDim.x * blockDim.x) {
    const int s = i / L.cap, j = i - s * L.cap;
    if (j < n_from[s]) {
      const EpMeta m = meta[i];
      ids_out[i] = m.expert;
      w_out[i] = m.weight;
      src_slot_out[i] = m.slot;
    } else {
      ids_out[i] = -1;
      w_out[i] = 0.f;
      src_slot_out[i] = -1;
    }
  }
}

// one warp per received row: copy the e4m3 row and transpose its scales into [kb][row]
__global__ void ep_scatter_q_kernel(EpLayout L, EpPeers peers, const int* __restrict__ ids, const int* __restrict__ pos,
                                    const float* __restrict__ w, const int* __restrict__ src_slot, int n,
                                    const int* __restrict__ seg_start, const int* __restrict__ seg_len, uint8_t* xq,
                                    float* xs, int xs_ld, float* row_w, int* row_src_rank, int* row_src_slot) {
  const int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (i >= n) return;
  const int e = ids[i];
  if (e < 0) return;
  const int ps = pos[i];
  if (ps < 0 || ps >= seg_len[e]) return;
  const int row = seg_start[e] + ps;
  unsigned char* self = peers.p[L.rank];
  const int H = L.H, nb = H >> 7;
  const size_t rb = (size_t)H * (L.payload == 2 ? 2 : 1);   // bytes per row
  const uint4* src = reinterpret_cast<const uint4*>(self + L.off_recv_x + (size_t)i * rb);
  uint4* dst = reinterpret_cast<uint4*>(xq + (size_t)row * rb);
  for (int c = lane; c < (int)(rb >> 4); c += 32) dst[c] = src[c];
  if (L.payload != 2) {
    const float* ss = reinterpret_cast<const float*>(self + L.off_recv_s) + (size_t)i * nb;
    for (int b = lane; b < nb; b += 32) xs[(size_t)b * xs_ld + row] = ss[b];
  }
  if (lane == 0) {
    row_w[row] = w[i];
    row_src_rank[row] = i / L.cap;
    row_src_slot[row] = src_slot[i];
  }
}

// one warp per expert-sorted row: y[row] -> comb[src_slot] on the source rank
__global__ void __launch_bounds__(256)
ep_combine_send_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ total_rows,
                       const int* __restrict__ seg_start, const int* __restrict__ seg_len, int e_local,
                       const int* __restrict__ row_src_rank, const int* __restrict__ row_src_slot, EpLayout L,
                       EpPeers peers) {
  unsigned char* self = peers.p[L.rank];
  int* ctrl = reinterpret_cast<int*>(self + L.off_ctrl);
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int H = L.H;
  const int rows = *total_rows;
  for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows; row += gridDim.x * warps_per_block) {
    // rows in the alignment gaps between expert segments carry no token
    bool live = false;
    for (int e = 0; e < e_local; ++e) {
      const int s0 = seg_start[e];
      if (row >= s0 && row < s0 + seg_len[e]) { live = true; break; }
      if (row < s0) break;
    }
    if (!live) continue;
    const int s = row_src_rank[row], slot = row_src_slot[row];
    if (s < 0 || s >= L.world || slot < 0 || slot >= L.max_slots) continue;
    const uint4* src = reinterpret_cast<const uint4*>(y + (size_t)row * H);
    uint4* dst = reinterpret_cast<uint4*>(peers.p[s] + L.off_comb + (size_t)slot * H * 2);
#pragma unroll 4
    for (int c = lane; c < (H >> 3); c += 32) dst[c] = src[c];
  }
  __threadfence_system();
  __syncthreads();
  __shared__ int is_last;
  if (threadIdx.x == 0) is_last = (atomicAdd(&ctrl[3], 1) == (int)gridDim.x - 1);
  __syncthreads();
  if (is_last) {
    __threadfence_system();
    const int epoch = ctrl[1] + 1;
    if ((int)threadIdx.x < L.world) {
      int* flag = reinterpret_cast<int*>(peers.p[threadIdx.x] + L.off_comb_flag);
      st_release_sys(&flag[L.rank], epoch);
    }
    __syncthreads();
    if (threadIdx.x == 0) { ctrl[1] = epoch; ctrl[3] = 0; }
  }
}

// one CTA per token
__global__ void ep_combine_reduce_kernel(EpLayout L, EpPeers peers, const int* __restrict__ ids, int n_tokens, int top_k,
                                         const __nv_bfloat16* __restrict__ shared, __nv_bfloat16* out,
                                         unsigned long long wait_ns, OmniStatus* status) {
  unsigned char* self = peers.p[L.rank];
  const int* ctrl = reinterpret_cast<const int*>(self + L.off_ctrl);
  const int* flag = reinterpret_cast<const int*>(self + L.off_comb_flag);
  const int epoch = ctrl[1];   // this rank's combine_send ran first on the same stream
  __shared__ int ok_all;
  if (threadIdx.x == 0) ok_all = 1;
  __syncthreads();
  if ((int)threadIdx.x < L.world) {
    if (!flag_wait_ge(&flag[threadIdx.x], epoch, wait_ns, status, 202, threadIdx.x)) ok_all = 0;
  }
  __syncthreads();
  const int t = blockIdx.x;
  if (t >= n_tokens) return;   // an idle rank still waits above so that epochs stay in step
  const int H = L.H;
  const __nv_bfloat16* comb = reinterpret_cast<const __nv_bfloat16*>(self + L.off_comb);
  // gridDim.y column parts per token: a decode batch has only a few hundred tokens, one CTA each leaves SMs idle
  const int part = (H / 8 + gridDim.y - 1) / gridDim.y * 8;
  const int c_lo = blockIdx.y * part, c_hi = min(H, c_lo + part);
  for (int c = c_lo + threadIdx.x * 8; c < c_hi; c += blockDim.x * 8) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    if (ok_all) {
#pragma unroll 4
      for (int k = 0; k < top_k; ++k) {
        if (ids[t * top_k + k] < 0) continue;
        uint4 raw = *reinterpret_cast<const uint4*>(comb + (size_t)(t * top_k + k) * H + c);
        const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += __bfloat162float(h[j]);
      }
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

// ---- symmetric buffer plumbing (CUDA IPC) ---------------------------------------------------------------
extern "C" int omni_symm_alloc(void** ptr, long long bytes) {
  cudaError_t e = cudaMalloc(ptr, (size_t)bytes);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaMemset(*ptr, 0, (size_t)bytes);
}
extern "C" int omni_symm_free(void* ptr) { return (int)cudaFree(ptr); }
extern "C" int omni_symm_get_handle(void* ptr, void* handle64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) return (int)e;
  memcpy(handle64, &h, sizeof(h));
  return 0;
}
extern "C" int omni_symm_open_handle(const void* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  return (int)cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
}
extern "C" int omni_symm_close_handle(void* ptr) { return (int)cudaIpcCloseMemHandle(ptr); }

static EpPeers make_peers(void* const* peer_ptrs, int world) {
  EpPeers p;
  for (int i = 0; i < 16; ++i) p.p[i] = (unsigned char*)(i < world ? peer_ptrs[i] : nullptr);
  return p;
}

// x: bf16 rows [T, H].  xq_in / xs_in (optional, e4m3 payload only): the same rows already quantised, scales K-block
// major [H/128, xs_in_ld]; then x may be null.
extern "C" int omni_ep_dispatch_send(const void* x, const void* xq_in, const float* xs_in, int xs_in_ld, const int* ids,
                                     const float* w, int T, int top_k, int slots_per_rank, const EpLayout* L,
                                     void* const* peer_ptrs, void* status, cudaStream_t stream) {
  if (L->world > 16 || (L->H % 128) != 0) return -1;
  if (x == nullptr && (xq_in == nullptr || L->payload == 2)) return -2;
  if (xq_in != nullptr && xs_in == nullptr) return -2;
  const int n = T * top_k;
  int blocks = (n + 7) / 8;
  if (blocks < 1) blocks = 1;
  if (blocks > 592) blocks = 592;
  ep_dispatch_send_kernel<<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, (const uint8_t*)xq_in, xs_in, xs_in_ld, ids, w, n,
                                                      top_k, slots_per_rank, *L, make_peers(peer_ptrs, L->world),
                                                      (OmniStatus*)status);
  return (int)cudaGetLastError();
}

extern "C" int omni_ep_dispatch_recv(const EpLayout* L, void* const* peer_ptrs, int* ids_out, float* w_out,
                                     int* src_slot_out, int* counts_out, unsigned long long wait_ns, void* status,
                                     cudaStream_t stream) {
  int blocks = (L->world * L->cap + 4095) / 4096;
  if (blocks < 1) blocks = 1;
  if (blocks > 32) blocks = 32;
  ep_dispatch_recv_kernel<<<blocks, 1024, 0, stream>>>(*L, make_peers(peer_ptrs, L->world), ids_out, w_out, src_slot_out,
                                                  counts_out, wait_ns, (OmniStatus*)status);
  return (int)cudaGetLastError();
}

extern "C" int omni_ep_scatter_q(const EpLayout* L, void* const* peer_ptrs, const int* ids, const int* pos,
                                 const float* w, const int* src_slot, const int* seg_start, const int* seg_len,
                                 void* xq, float* xs, int xs_ld, float* row_w, int* row_src_rank, int* row_src_slot,
                                 cudaStream_t stream) {
  const int n = L->world * L->cap;
  const long long threads = (long long)n * 32;
  ep_scatter_q_kernel<<<(int)((threads + 255) / 256), 256, 0, stream>>>(
      *L, make_peers(peer_ptrs, L->world), ids, pos, w, src_slot, n, seg_start, seg_len, (uint8_t*)xq, xs, xs_ld, row_w,
      row_src_rank, row_src_slot);
  return (int)cudaGetLastError();
}

extern "C" int omni_ep_combine_send(const void* y, const int* total_rows, const int* seg_start, const int* seg_len,
                                    int e_local, const int* row_src_rank, const int* row_src_slot, int max_rows,
                                    const EpLayout* L, void* const* peer_ptrs, cudaStream_t stream) {
  int blocks = (max_rows + 7) / 8;
  if (blocks < 1) blocks = 1;
  if (blocks > 592) blocks = 592;
  ep_combine_send_kernel<<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)y, total_rows, seg_start, seg_len, e_local,
                                                     row_src_rank, row_src_slot, *L, make_peers(peer_ptrs, L->world));
  return (int)cudaGetLastError();
}

extern "C" int omni_ep_combine_reduce(const EpLayout* L, void* const* peer_ptrs, const int* ids, int T, int top_k,
                                      const void* shared, void* out, unsigned long long wait_ns, void* status,
                                      cudaStream_t stream) {
  int parts = 1;
  while (T * parts < 1184 && parts < 8 && L->H / (parts * 2) >= 512) parts *= 2;   // aim at 8 CTAs per SM
  int threads = (L->H / parts + 7) / 8;
  threads = (threads + 31) / 32 * 32;
  if (threads > 256) threads = 256;
  if (threads < 32) threads = 32;
  ep_combine_reduce_kernel<<<dim3(T > 0 ? T : 1, parts), threads, 0, stream>>>(*L, make_peers(peer_ptrs, L->world), ids, T, top_k,
                                                      (const __nv_bfloat16*)shared, (__nv_bfloat16*)out, wait_ns,
                                                      (OmniStatus*)status);
  return (int)cudaGetLastError();
}
