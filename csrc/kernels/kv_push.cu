// Prefill -> decode KV-cache push: copies paged-cache blocks of a finished prefill request from this GPU's
// cache into the decode instance's paged cache through NVLink peer memory (the destination pointers are the
// decode GPU's cache tensors opened with CUDA IPC).  One CTA per (layer tensor, block); 16-byte vector copies;
// a system-scope fence before the completion counter is bumped so that the host-side "done" message is only sent
// after the data is visible on the peer.  Also used for the expert-weight swap of the placement engine
// (contiguous copy with n_tensors = 1).
//
// The reference pulls blocks with its vendor transfer library (omni/accelerators/pd/llmdatadist_manager.py:185-215);
// on one NVSwitch box a push kernel into peer memory does the same job without a transfer service.
#include "../include/omni_ptx.cuh"

namespace omni {

struct KvPushParams {
  const unsigned char* const* src;   // [n_tensors] base pointers of the local cache tensors
  unsigned char* const* dst;         // [n_tensors] base pointers of the peer cache tensors
  const long long* src_block;        // [n_blocks]
  const long long* dst_block;        // [n_blocks]
  long long block_bytes;             // bytes of one block in one tensor (multiple of 16)
  long long src_blocks_total, dst_blocks_total;   // bounds
  int n_tensors, n_blocks;
  int* done_counter;                 // optional: incremented once per CTA
  OmniStatus* status;
};

__global__ void __launch_bounds__(256) kv_push_kernel(const KvPushParams p) {
  const int t = blockIdx.y, b = blockIdx.x;
  const long long sb = p.src_block[b], db = p.dst_block[b];
  if (sb < 0 || sb >= p.src_blocks_total || db < 0 || db >= p.dst_blocks_total) {
    if (threadIdx.x == 0) report_status(p.status, OMNI_ERR_BOUNDS, 300, b);
    return;
  }
  const uint4* s = reinterpret_cast<const uint4*>(p.src[t] + sb * p.block_bytes);
  uint4* d = reinterpret_cast<uint4*>(p.dst[t] + db * p.block_bytes);
  const long long n16 = p.block_bytes >> 4;
  for (long long i = threadIdx.x; i < n16; i += blockDim.x) d[i] = s[i];
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0 && p.done_counter) atomicAdd_system(p.done_counter, 1);
}

}  // namespace omni

using namespace omni;

// src_ptrs / dst_ptrs / src_block / dst_block are DEVICE arrays.
extern "C" int omni_kv_push(const void* const* src_ptrs, void* const* dst_ptrs, const long long* src_block,
                            const long long* dst_block, long long block_bytes, long long src_blocks_total,
                            long long dst_blocks_total, int n_tensors, int n_blocks, int* done_counter, void* status,
                            cudaStream_t stream) {
  if (n_tensors <= 0 || n_blocks <= 0) return 0;
  if (block_bytes % 16 != 0) return -1;
  KvPushParams p;
  p.src = (const unsigned char* const*)src_ptrs; p.dst = (unsigned char* const*)dst_ptrs;
  p.src_block = src_block; p.dst_block = dst_block; p.block_bytes = block_bytes;
  p.src_blocks_total = src_blocks_total; p.dst_blocks_total = dst_blocks_total;
  p.n_tensors = n_tensors; p.n_blocks = n_blocks; p.done_counter = done_counter; p.status = (OmniStatus*)status;
  dim3 grid(n_blocks, n_tensors);
  kv_push_kernel<<<grid, 256, 0, stream>>>(p);
  return (int)cudaGetLastError();
}
