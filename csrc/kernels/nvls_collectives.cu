// Collectives that reduce inside the NVSwitch (NVLS): `multimem.ld_reduce` on a multicast address returns the sum of
// the same location on every GPU bound to the multicast object, `multimem.st` writes a value to all of them.  Data of
// an all-reduce therefore crosses every link once in each direction, and the additions happen in the switch.
//
//   omni_nvls_allreduce      in place on a symmetric buffer [numel] bf16: rank r reduces the r-th part of every
//                            strip with ld_reduce and broadcasts the sums with multimem.st (two-shot through the switch)
//   omni_nvls_reduce_rows    reduce-scatter form used after a row-parallel GEMM: every rank has written its partial
//                            [rows_total, n] into its own symmetric buffer; this rank pulls the sums of its row block,
//                            optionally adds the residual stream and applies RMSNorm in the same pass (the multimem
//                            counterpart of rs_reduce_kernel in tp_fused.cu, which adds slabs written by peer stores)
//
// Entry and exit are guarded by a flag barrier over the ranks' symmetric buffers (one flag word per peer in the tail of
// the buffer).  The round counter lives in device memory and advances inside the kernel, so a captured CUDA graph
// replays correctly.  Every wait is bounded; when one runs out the kernel records it in the
// status word and returns without touching the data.
//
// The multicast and peer addresses come from the host (torch symmetric memory rendezvous); nothing here binds or
// unbinds multicast memory.  Stands where the reference calls tensor_model_parallel_all_reduce / reduce_scatter
// (omni/adaptors/vllm/distributed/communication_op.py).
#include "../include/omni_ptx.cuh"

#include <cuda_bf16.h>

namespace omni {

enum { NVS_BARRIER_IN = 51, NVS_BARRIER_OUT = 52 };

struct NvlsParams {
  uint8_t* mc;             // multicast address of the symmetric buffer
  uint8_t* local;          // this rank's own mapping of it
  int* peer_flags[8];      // per rank: base of its flag block (2 x 8 ints: entry flags, exit flags)
  int* done;               // local CTA counter (inside the local flag block, word 16)
  int* epoch;              // local round counter (word 17): rounds completed so far; this call runs round *epoch + 1
  int world, rank;
  long long numel;         // bf16 elements (all-reduce) / rows_total * n (reduce rows)
  unsigned long long wait_ns;
  OmniStatus* status;
  // reduce_rows only
  int rows_per_rank, n;
  const __nv_bfloat16* residual_in;
  __nv_bfloat16* sum_out;
  const __nv_bfloat16* norm_weight;
  __nv_bfloat16* norm_out;
  float eps;
};

__device__ __forceinline__ void mm_ld_reduce_bf16x8(const void* mc_addr, uint32_t (&v)[4]) {
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3])
               : "l"(mc_addr)
               : "memory");
}
__device__ __forceinline__ void mm_st_bf16x8(void* mc_addr, const uint32_t (&v)[4]) {
  asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "r"(v[0]), "r"(v[1]),
               "r"(v[2]), "r"(v[3])
               : "memory");
}

// Every CTA: read the round, wait until every rank has published it in this rank's entry flags.  CTA 0 publishes
// first.  s_state[0] = all flags seen, s_state[1] = the round.
__device__ __forceinline__ bool nvls_enter(const NvlsParams& p, int* s_state) {
  if (threadIdx.x == 0) { s_state[0] = 1; s_state[1] = *reinterpret_cast<volatile int*>(p.epoch) + 1; }
  __syncthreads();
  const int round = s_state[1];
  if (blockIdx.x == 0 && (int)threadIdx.x < p.world) {
    __threadfence_system();   // this rank's partial sums (written by the kernel before this one) are visible to the fabric
    st_release_sys(p.peer_flags[threadIdx.x] + p.rank, round);
  }
  if ((int)threadIdx.x < p.world) {
    if (!flag_wait_ge(p.peer_flags[p.rank] + threadIdx.x, round, p.wait_ns, p.status, NVS_BARRIER_IN, threadIdx.x)) s_state[0] = 0;
  }
  __syncthreads();
  return s_state[0] != 0;
}

// Last CTA of the grid: publish "my multicast stores are done" and wait for everybody's, so that the kernel that
// follows on any rank sees all sums.  (reduce_rows has no multicast stores: its exit only tells the peers that their
// buffers may be overwritten by the next round.)
// Every CTA arrives here, also one whose entry wait ran out (the CTA counter and the round must stay in step with
// the other ranks' for the calls that follow).
__device__ __forceinline__ void nvls_exit(const NvlsParams& p, const int* s_state) {
  __threadfence_system();
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) s_last = (atomicAdd(p.done, 1) == (int)gridDim.x - 1);
  __syncthreads();
  if (!s_last) return;
  const int round = s_state[1];
  if ((int)threadIdx.x < p.world) {
    st_release_sys(p.peer_flags[threadIdx.x] + 8 + p.rank, round);
    if (s_state[0]) flag_wait_ge(p.peer_flags[p.rank] + 8 + threadIdx.x, round, p.wait_ns, p.status, NVS_BARRIER_OUT, threadIdx.x);
  }
  __syncthreads();
  if (threadIdx.x == 0) { *p.done = 0; *p.epoch = round; }   // every CTA read the round before it arrived here
}

__global__ void __launch_bounds__(512) nvls_allreduce_kernel(const NvlsParams p) {
  __shared__ int s_state[2];
  if (!nvls_enter(p, s_state)) { nvls_exit(p, s_state); return; }
  // strips of world * 8 elements per thread step: rank r owns the r-th 16-byte vector of every strip, so consecutive
  // threads of one rank touch addresses world * 16 bytes apart and all ranks together cover the buffer densely
  const long long vecs = p.numel / 8;
  const long long mine = (vecs + p.world - 1 - p.rank) / p.world;     // vectors v with v % world == rank
  // four reductions in flight per thread before the first broadcast: the round trip through the switch is long and a
  // thread that waits for each sum before asking for the next leaves the links idle
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + 3 * stride < mine; i += 4 * stride) {
    uint32_t r[4][4];
#pragma unroll
    for (int u = 0; u < 4; ++u) mm_ld_reduce_bf16x8(p.mc + ((i + u * stride) * p.world + p.rank) * 16, r[u]);
#pragma unroll
    for (int u = 0; u < 4; ++u) mm_st_bf16x8(p.mc + ((i + u * stride) * p.world + p.rank) * 16, r[u]);
  }
  for (; i < mine; i += stride) {
    const long long v = i * p.world + p.rank;
    uint32_t r[4];
    mm_ld_reduce_bf16x8(p.mc + v * 16, r);
    mm_st_bf16x8(p.mc + v * 16, r);
  }
  nvls_exit(p, s_state);
}

// one CTA per row of this rank's block
__global__ void __launch_bounds__(256) nvls_reduce_rows_kernel(const NvlsParams p) {
  __shared__ int s_state[2];
  __shared__ float s_part[8];
  if (!nvls_enter(p, s_state)) { nvls_exit(p, s_state); return; }
  const int nv = p.n / 8;
  for (int row = blockIdx.x; row < p.rows_per_rank; row += gridDim.x) {
    const long long grow = (long long)p.rank * p.rows_per_rank + row;
    float ssq = 0.f;
    for (int v = threadIdx.x; v < nv; v += blockDim.x) {
      uint32_t r[4];
      mm_ld_reduce_bf16x8(p.mc + (grow * p.n + (long long)v * 8) * 2, r);
      float acc[8];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(r);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        acc[2 * e] = f.x;
        acc[2 * e + 1] = f.y;
      }
      if (p.residual_in) {
        const uint4 u = *reinterpret_cast<const uint4*>(p.residual_in + (long long)row * p.n + v * 8);
        const __nv_bfloat162* hr = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(hr[e]);
          acc[2 * e] += f.x;
          acc[2 * e + 1] += f.y;
        }
      }
      __nv_bfloat162 o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        o[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
        const float2 f = __bfloat1622float2(o[e]);     // the norm sees the rounded sum, as the unfused sequence does
        ssq += f.x * f.x + f.y * f.y;
      }
      *reinterpret_cast<uint4*>(p.sum_out + (long long)row * p.n + v * 8) = *reinterpret_cast<const uint4*>(o);
    }
    if (p.norm_weight) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
      if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ssq;
      __syncthreads();
      float tot = 0.f;
      for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += s_part[w];
      const float inv = rsqrtf(tot / (float)p.n + p.eps);
      for (int v = threadIdx.x; v < nv; v += blockDim.x) {
        const uint4 u = *reinterpret_cast<const uint4*>(p.sum_out + (long long)row * p.n + v * 8);
        const uint4 wv = *reinterpret_cast<const uint4*>(p.norm_weight + v * 8);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
        const __nv_bfloat162* hw = reinterpret_cast<const __nv_bfloat162*>(&wv);
        __nv_bfloat162 o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(h[e]), g = __bfloat1622float2(hw[e]);
          o[e] = __floats2bfloat162_rn(f.x * inv * g.x, f.y * inv * g.y);
        }
        *reinterpret_cast<uint4*>(p.norm_out + (long long)row * p.n + v * 8) = *reinterpret_cast<const uint4*>(o);
      }
      __syncthreads();   // s_part is reused by the next row
    }
  }
  nvls_exit(p, s_state);
}

}  // namespace omni

using namespace omni;

static int fill_common(NvlsParams& p, void* mc, void* local, void* const* peer_bufs, long long flag_offset, int world, int rank,
                       unsigned long long wait_ns, void* status) {
  if (world < 1 || world > 8 || rank < 0 || rank >= world || mc == nullptr || local == nullptr) return -1;
  if (flag_offset % 16 != 0) return -2;
  p.mc = (uint8_t*)mc;
  p.local = (uint8_t*)local;
  for (int i = 0; i < 8; ++i) p.peer_flags[i] = i < world ? (int*)((uint8_t*)peer_bufs[i] + flag_offset) : nullptr;
  p.done = p.peer_flags[rank] + 16;
  p.epoch = p.peer_flags[rank] + 17;
  p.world = world; p.rank = rank; p.wait_ns = wait_ns; p.status = (OmniStatus*)status;
  return 0;
}

// Symmetric buffer layout expected by both entry points: [data][flag block of 128 bytes at `flag_offset`: 8 entry flags,
// 8 exit flags, the CTA counter, the round counter], zeroed once at allocation.  `peer_bufs[r]` is rank r's buffer as mapped into this process; `mc` the multicast mapping.
extern "C" int omni_nvls_allreduce(void* mc, void* local, void* const* peer_bufs, long long flag_offset, int world, int rank,
                                   long long numel, int ctas, unsigned long long wait_ns, void* status, cudaStream_t stream) {
  NvlsParams p = {};
  if (int e = fill_common(p, mc, local, peer_bufs, flag_offset, world, rank, wait_ns, status)) return e;
  if (numel <= 0 || numel % 8 != 0 || numel * 2 > flag_offset) return -3;
  p.numel = numel;
  const long long mine = (numel / 8 + world - 1) / world;
  // small messages: few CTAs (every CTA polls the entry flags); large ones: enough threads to keep four vectors per
  // thread in flight on every link, at most one CTA per SM
  int grid = (int)((mine + 2047) / 2048);
  if (grid < 1) grid = 1;
  const int cap = ctas > 0 ? ctas : 148;
  if (grid > cap) grid = cap;
  nvls_allreduce_kernel<<<grid, 512, 0, stream>>>(p);
  return (int)cudaGetLastError();
}

extern "C" int omni_nvls_reduce_rows(void* mc, void* local, void* const* peer_bufs, long long flag_offset, int world, int rank,
                                     int rows_per_rank, int n, const void* residual_in, void* sum_out,
                                     const void* norm_weight, void* norm_out, float eps, unsigned long long wait_ns,
                                     void* status, cudaStream_t stream) {
  NvlsParams p = {};
  if (int e = fill_common(p, mc, local, peer_bufs, flag_offset, world, rank, wait_ns, status)) return e;
  if (rows_per_rank <= 0 || n <= 0 || n % 8 != 0 || (long long)rows_per_rank * world * n * 2 > flag_offset) return -3;
  if (norm_weight != nullptr && norm_out == nullptr) return -4;
  p.rows_per_rank = rows_per_rank; p.n = n; p.numel = (long long)rows_per_rank * world * n;
  p.residual_in = (const __nv_bfloat16*)residual_in; p.sum_out = (__nv_bfloat16*)sum_out;
  p.norm_weight = (const __nv_bfloat16*)norm_weight; p.norm_out = (__nv_bfloat16*)norm_out; p.eps = eps;
  const int grid = rows_per_rank < 592 ? rows_per_rank : 592;
  nvls_reduce_rows_kernel<<<grid, 256, 0, stream>>>(p);
  return (int)cudaGetLastError();
}
