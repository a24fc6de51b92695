// Tensor-parallel collectives that bracket the fused GEMMs of gemm_tokmajor_sm100.cu, over peer memory.
//
//   omni_ag_push    all-gather, producer side: copy this rank's row block into every rank's gather buffer (its own
//                   included) with 16-byte peer stores, then publish "block of rank r, round e has landed" on every
//                   rank.  The GEMM that follows on each rank waits per source block, so it starts on its own rows
//                   while the others are still in flight.
//   omni_ag_collect plain all-gather, consumer side: wait (bounded) for every rank's block of the current round, then
//                   copy the gathered rows out of the receive buffer.  The receive buffer has two halves used in
//                   turn (chosen by the round counter in device memory), so a rank that is already pushing the next
//                   round cannot overwrite rows a slower rank is still copying.
//   omni_rs_reduce  reduce-scatter, consumer side: the GEMM epilogues of all ranks have written their partial rows
//                   into this rank's slab [source rank][row][n]; wait (bounded) for every source's flag, add the
//                   slabs in fp32, optionally add the residual stream and apply RMSNorm in the same pass.
//
// Flags and round counters live in device memory and advance inside the kernels, so a captured CUDA graph replays
// correctly.  Every wait has a time limit; when it runs out the kernel records where in the status word and returns.
//
// Stand where the reference calls tensor_model_parallel_all_gather / reduce_scatter around the attention block
// (omni/models/common/layers/attention/deepseek_mla.py:437-470, omni/adaptors/vllm/distributed/communication_op.py).
#include "../include/omni_ptx.cuh"

#include <cuda_bf16.h>

namespace omni {

enum { TPS_RS_FLAG = 41 };

struct AgPushParams {
  const uint8_t* src;      // [rows, row_bytes] this rank's block
  int rows, row_bytes;     // row_bytes a multiple of 16
  long long dst_row_pitch; // bytes between rows of the gather buffers
  long long dst_offset;    // byte offset of this rank's block inside every gather buffer
  long long parity_stride; // != 0: the gather buffers have two halves this far apart, rounds alternate between them
  int world, rank, signal;
  uint8_t* gather[8];      // per rank: base of its gather buffer
  int* flag[8];            // per rank: flag word of this source rank
  int* epoch;              // local round counter (advanced here)
  int* done;               // local CTA counter
};

__global__ void ag_push_kernel(const AgPushParams p) {
  const int vec_per_row = p.row_bytes / 16;
  const long long total = (long long)p.rows * vec_per_row;
  const long long half = p.parity_stride ? (long long)((*p.epoch + 1) & 1) * p.parity_stride : 0;   // round being produced
  __syncthreads();   // every thread has read the round counter before the last CTA advances it
  for (int d0 = 0; d0 < p.world; ++d0) {
    const int d = (p.rank + 1 + d0) % p.world;   // remote ranks first, the local copy last
    uint8_t* dst = p.gather[d] + p.dst_offset + half;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
      const int r = (int)(i / vec_per_row), c = (int)(i - (long long)r * vec_per_row);
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(p.src + (long long)r * p.row_bytes) + c);
      *(reinterpret_cast<uint4*>(dst + (long long)r * p.dst_row_pitch) + c) = v;
    }
  }
  if (!p.signal) return;   // a later push on the same stream publishes the flag that covers these rows too
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int done = atomicAdd(p.done, 1);
    if (done == (int)gridDim.x - 1) {
      *p.done = 0;
      const int round = *p.epoch + 1;
      *p.epoch = round;
      __threadfence_system();
      for (int d = 0; d < p.world; ++d) st_release_sys(p.flag[d], round);
    }
  }
}

struct RsReduceParams {
  const __nv_bfloat16* slab;   // [world][rows_per_rank][ld]
  long long parity_stride;     // elements; != 0: two halves used in turn, the current one is (round & 1)
  int world, rows, n, ld;
  long long src_pitch;         // elements between source slabs
  const int* flag;             // [world]
  const int* epoch;            // local round counter (already advanced by this rank's GEMM)
  unsigned long long wait_ns;
  const __nv_bfloat16* residual_in;   // optional [rows, n]
  __nv_bfloat16* sum_out;             // [rows, n] sum (+ residual)
  const __nv_bfloat16* norm_weight;   // optional [n]
  __nv_bfloat16* norm_out;            // [rows, n] when norm_weight is given
  float eps;
  OmniStatus* status;
};

// one CTA per row; n <= 8 * 1024 * 2 handled by striding
__global__ void __launch_bounds__(256) rs_reduce_kernel(const RsReduceParams p) {
  __shared__ int s_ok;
  __shared__ float s_part[8];
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < p.world) {
    const int round = *p.epoch;
    if (!flag_wait_ge(p.flag + threadIdx.x, round, p.wait_ns, p.status, TPS_RS_FLAG, threadIdx.x)) s_ok = 0;
  }
  __syncthreads();
  if (!s_ok) return;
  const int row = blockIdx.x;
  if (row >= p.rows) return;
  const int nv = p.n / 8;
  const __nv_bfloat16* slab = p.slab + (p.parity_stride ? (long long)(*p.epoch & 1) * p.parity_stride : 0);
  float ssq = 0.f;
  for (int v = threadIdx.x; v < nv; v += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < p.world; ++s) {
      const uint4 u = *reinterpret_cast<const uint4*>(slab + (long long)s * p.src_pitch + (long long)row * p.ld + v * 8);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        acc[2 * e] += f.x;
        acc[2 * e + 1] += f.y;
      }
    }
    if (p.residual_in) {
      const uint4 u = *reinterpret_cast<const uint4*>(p.residual_in + (long long)row * p.n + v * 8);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        acc[2 * e] += f.x;
        acc[2 * e + 1] += f.y;
      }
    }
    __nv_bfloat162 o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      o[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
      const float2 f = __bfloat1622float2(o[e]);   // the norm sees what the residual stream stores
      ssq += f.x * f.x + f.y * f.y;
    }
    *reinterpret_cast<uint4*>(p.sum_out + (long long)row * p.n + v * 8) = *reinterpret_cast<uint4*>(o);
  }
  if (p.norm_weight == nullptr) return;
  ssq = warp_sum(ssq);
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ssq;
  __syncthreads();
  float tot = 0.f;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += s_part[w];
  const float inv = rsqrtf(tot / (float)p.n + p.eps);
  for (int v = threadIdx.x; v < nv; v += blockDim.x) {
    const uint4 u = *reinterpret_cast<const uint4*>(p.sum_out + (long long)row * p.n + v * 8);
    const uint4 wv = *reinterpret_cast<const uint4*>(p.norm_weight + v * 8);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
    const __nv_bfloat162* wh = reinterpret_cast<const __nv_bfloat162*>(&wv);
    __nv_bfloat162 o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __bfloat1622float2(h[e]);
      const float2 g = __bfloat1622float2(wh[e]);
      o[e] = __floats2bfloat162_rn(f.x * inv * g.x, f.y * inv * g.y);
    }
    *reinterpret_cast<uint4*>(p.norm_out + (long long)row * p.n + v * 8) = *reinterpret_cast<uint4*>(o);
  }
}

struct AgCollectParams {
  const uint8_t* gather;   // local receive buffer (two halves)
  long long parity_stride;
  uint8_t* dst;
  long long bytes;         // multiple of 16
  int world;
  const int* flag;         // [world]
  const int* epoch;        // local round counter (already advanced by this rank's push)
  unsigned long long wait_ns;
  OmniStatus* status;
};

__global__ void __launch_bounds__(256) ag_collect_kernel(const AgCollectParams p) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  const int round = *p.epoch;
  if (threadIdx.x < p.world) {
    if (!flag_wait_ge(p.flag + threadIdx.x, round, p.wait_ns, p.status, TPS_RS_FLAG + 1, threadIdx.x)) s_ok = 0;
  }
  __syncthreads();
  if (!s_ok) return;
  const uint8_t* src = p.gather + (long long)(round & 1) * p.parity_stride;
  const long long nv = p.bytes / 16;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += (long long)gridDim.x * blockDim.x)
    reinterpret_cast<uint4*>(p.dst)[i] = reinterpret_cast<const uint4*>(src)[i];
}

}  // namespace omni

using namespace omni;

extern "C" int omni_ag_collect(const void* gather, long long parity_stride, void* dst, long long bytes, int world,
                               const int* flag, const int* epoch, unsigned long long wait_ns, void* status,
                               cudaStream_t stream) {
  if (world < 1 || world > 8 || (bytes % 16) != 0 || (parity_stride % 16) != 0 || epoch == nullptr || flag == nullptr) return -1;
  AgCollectParams p;
  p.gather = (const uint8_t*)gather; p.parity_stride = parity_stride; p.dst = (uint8_t*)dst; p.bytes = bytes; p.world = world;
  p.flag = flag; p.epoch = epoch; p.wait_ns = wait_ns; p.status = (OmniStatus*)status;
  long long nv = bytes / 16;
  int grid = (int)((nv + 255) / 256);
  if (grid < 1) grid = 1;
  if (grid > 148) grid = 148;
  ag_collect_kernel<<<grid, 256, 0, stream>>>(p);
  return (int)cudaGetLastError();
}

// Copies [rows, row_bytes] from `src` to byte offset `dst_offset` (row pitch `dst_row_pitch`) of every rank's
// gather buffer.  With signal != 0 the last CTA then advances this rank's round counter and writes it to this
// rank's flag word on every rank.
extern "C" int omni_ag_push(const void* src, int rows, int row_bytes, long long dst_row_pitch, long long dst_offset,
                            long long parity_stride, int world, int rank, int signal, void* const* gather,
                            int* const* flag, int* epoch, int* done, cudaStream_t stream) {
  if (parity_stride != 0 && (!signal || (parity_stride % 16) != 0)) return -4;
  if (world < 1 || world > 8 || rows < 0 || (row_bytes % 16) != 0 || (dst_row_pitch % 16) != 0 || (dst_offset % 16) != 0) return -1;
  if (signal && (epoch == nullptr || done == nullptr)) return -2;
  AgPushParams p;
  p.src = (const uint8_t*)src; p.rows = rows; p.row_bytes = row_bytes; p.dst_row_pitch = dst_row_pitch;
  p.world = world; p.rank = rank; p.signal = signal; p.dst_offset = dst_offset; p.parity_stride = parity_stride; p.epoch = epoch; p.done = done;
  for (int d = 0; d < world; ++d) {
    if (gather[d] == nullptr || (signal && flag[d] == nullptr) || ((uintptr_t)gather[d] % 16) != 0) return -3;
    p.gather[d] = (uint8_t*)gather[d];
    p.flag[d] = signal ? flag[d] : nullptr;
  }
  const long long total = (long long)rows * (row_bytes / 16);
  int grid = (int)((total + 255) / 256);
  if (grid < 1) grid = 1;
  if (grid > 148) grid = 148;
  ag_push_kernel<<<grid, 256, 0, stream>>>(p);
  return (int)cudaGetLastError();
}

// parity_bytes != 0: the slab has two halves that far apart, used in turn; the current one is (round & 1).
extern "C" int omni_rs_reduce2(const void* slab, long long parity_bytes, int world, int rows, int n, int ld, long long src_pitch,
                               const int* flag, const int* epoch, unsigned long long wait_ns, const void* residual_in,
                               void* sum_out, const void* norm_weight, void* norm_out, float eps, void* status,
                               cudaStream_t stream);

extern "C" int omni_rs_reduce(const void* slab, int world, int rows, int n, int ld, long long src_pitch, const int* flag,
                              const int* epoch, unsigned long long wait_ns, const void* residual_in, void* sum_out,
                              const void* norm_weight, void* norm_out, float eps, void* status, cudaStream_t stream) {
  return omni_rs_reduce2(slab, 0, world, rows, n, ld, src_pitch, flag, epoch, wait_ns, residual_in, sum_out, norm_weight,
                         norm_out, eps, status, stream);
}

extern "C" int omni_rs_reduce2(const void* slab, long long parity_bytes, int world, int rows, int n, int ld, long long src_pitch,
                               const int* flag, const int* epoch, unsigned long long wait_ns, const void* residual_in,
                               void* sum_out, const void* norm_weight, void* norm_out, float eps, void* status,
                               cudaStream_t stream) {
  if (world < 1 || world > 8 || rows < 0 || (n % 8) != 0 || (ld % 8) != 0 || (src_pitch % 8) != 0 || (parity_bytes % 16) != 0) return -1;
  if (norm_weight != nullptr && norm_out == nullptr) return -2;
  RsReduceParams p;
  p.slab = (const __nv_bfloat16*)slab; p.parity_stride = parity_bytes / 2; p.world = world; p.rows = rows; p.n = n; p.ld = ld; p.src_pitch = src_pitch;
  p.flag = flag; p.epoch = epoch; p.wait_ns = wait_ns; p.residual_in = (const __nv_bfloat16*)residual_in;
  p.sum_out = (__nv_bfloat16*)sum_out; p.norm_weight = (const __nv_bfloat16*)norm_weight;
  p.norm_out = (__nv_bfloat16*)norm_out; p.eps = eps; p.status = (OmniStatus*)status;
  rs_reduce_kernel<<<rows > 0 ? rows : 1, 256, 0, stream>>>(p);   // an idle rank still launches (same sequence on every rank)
  return (int)cudaGetLastError();
}
