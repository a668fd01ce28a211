// Multi-destination copy over peer memory: the all-gather step of batch-sharded inference as one kernel of this
// library.  Every rank holds its slice of the output; the kernel reads each 16-byte vector of the slice once and stores
// it at the same offset of up to eight destination buffers - the rank's own copy of the gathered batch and, through
// peer pointers (NVLink / NVSwitch), every other rank's.  Plain stores only: no TMA, no multicast.  The reference has
// no distributed code; this stands where a batch of llc_run outputs computed on several GPUs is put together.
#include "common.cuh"

namespace llc {
namespace {

struct PushArgs {
  const uint4* src;
  uint4* dst[8];
  int nDst;
  long long vecs;          // 16-byte vectors
  const unsigned char* srcTail; unsigned char* dstTail[8]; int tail;   // the last bytes, fewer than 16
};

__global__ void __launch_bounds__(256) push_rows_kernel(const PushArgs a) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < a.vecs; i += stride * 4) {
    // four independent vectors per trip: the loads are issued before the first store
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) if (i + u * stride < a.vecs) v[u] = a.src[i + u * stride];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (i + u * stride < a.vecs) {
#pragma unroll
        for (int d = 0; d < 8; ++d) if (d < a.nDst) a.dst[d][i + u * stride] = v[u];
      }
  }
  if (blockIdx.x == 0 && (int)threadIdx.x < a.tail)
    for (int d = 0; d < a.nDst; ++d) a.dstTail[d][threadIdx.x] = a.srcTail[threadIdx.x];
  __threadfence_system();   // the stores have left for the peers before whatever the stream runs next (a barrier) signals them
}

}  // namespace
}  // namespace llc

using namespace llc;

extern "C" int llc_cuda_push_rows(const void* src, void* const* dst, int32_t n_dst, int64_t dst_offset_bytes, int64_t bytes, void* stream) {
  if (bytes <= 0 || n_dst <= 0) return LLC_OK;
  if (!src || !dst) return setError(LLC_ERR_ARGUMENT, "llc_cuda_push_rows: null pointer");
  if (n_dst > 8) return setError(LLC_ERR_UNSUPPORTED, "llc_cuda_push_rows: at most 8 destinations");
  if (dst_offset_bytes < 0 || dst_offset_bytes % 16 || reinterpret_cast<uintptr_t>(src) % 16)
    return setError(LLC_ERR_ARGUMENT, "llc_cuda_push_rows: source and destination offset must be 16-byte aligned");
  PushArgs a{};
  a.src = static_cast<const uint4*>(src);
  a.nDst = n_dst;
  a.vecs = bytes / 16;
  a.tail = (int)(bytes % 16);
  a.srcTail = static_cast<const unsigned char*>(src) + a.vecs * 16;
  for (int d = 0; d < n_dst; ++d) {
    if (!dst[d] || reinterpret_cast<uintptr_t>(dst[d]) % 16) return setError(LLC_ERR_ARGUMENT, "llc_cuda_push_rows: destinations must be 16-byte aligned");
    unsigned char* base = static_cast<unsigned char*>(dst[d]) + dst_offset_bytes;
    a.dst[d] = reinterpret_cast<uint4*>(base);
    a.dstTail[d] = base + a.vecs * 16;
  }
  const long long threads = (a.vecs + 3) / 4;
  long long blocks = (threads + 255) / 256;
  const long long cap = (long long)deviceSMs() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  push_rows_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  LLC_LAUNCH_CHECK("push_rows_kernel");
  return LLC_OK;
}
