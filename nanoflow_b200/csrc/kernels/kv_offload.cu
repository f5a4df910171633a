// Page gather / scatter between one layer's paged KV pool and a contiguous staging buffer, used by
// the layer-by-layer offload of retired requests (gather -> D2H on a copy stream) and by the reload
// path (H2D -> scatter). A small fixed CTA budget keeps it out of the way of the GEMMs it overlaps.
//
// Counterpart in the reference: moveKVcacheKernel, pipeline/src/offloadKernel.cu:16-35 (8 blocks x
// 256 threads, float4 copies), driven by PageAggregator / PageDispatcher (pipeline/include/otherWrapper.cuh:443-504).
#include "common.cuh"
#include "kernels.h"

namespace nf {
namespace {

__global__ void __launch_bounds__(256)
kv_move_pages_kernel(uint4* pool, uint4* staging, const int* __restrict__ page_ids, int n_pages,
                     long long vec_per_page, int num_pages, int direction, unsigned int* status) {
  for (int i = blockIdx.x; i < n_pages; i += gridDim.x) {
    const int page = page_ids[i];
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0) report_status(status, NF_ST_BAD_INDEX);
      continue;
    }
    uint4* pp = pool + static_cast<long long>(page) * vec_per_page;
    uint4* sp = staging + static_cast<long long>(i) * vec_per_page;
    if (direction == 0) {
      for (long long v = threadIdx.x; v < vec_per_page; v += blockDim.x) sp[v] = pp[v];
    } else {
      for (long long v = threadIdx.x; v < vec_per_page; v += blockDim.x) pp[v] = sp[v];
    }
  }
}

}  // namespace
}  // namespace nf

extern "C" int nfk_kv_move_pages(void* pool, void* staging, const int* page_ids, int n_pages,
                                 long long page_bytes, int num_pages, int direction, int num_ctas,
                                 unsigned int* status, cudaStream_t stream) {
  using namespace nf;
  if (n_pages == 0) return NF_OK;
  if (!pool || !staging || !page_ids || n_pages < 0 || page_bytes <= 0 || page_bytes % 16 != 0 ||
      num_pages <= 0 || (direction != 0 && direction != 1) ||
      (reinterpret_cast<uintptr_t>(pool) & 15) || (reinterpret_cast<uintptr_t>(staging) & 15))
    return NF_ERR_BAD_ARG;
  int ctas = num_ctas > 0 ? num_ctas : 8;
  if (ctas > n_pages) ctas = n_pages;
  kv_move_pages_kernel<<<ctas, 256, 0, stream>>>(reinterpret_cast<uint4*>(pool),
                                                 reinterpret_cast<uint4*>(staging), page_ids, n_pages,
                                                 page_bytes / 16, num_pages, direction, status);
  return cudaGetLastError() == cudaSuccess ? NF_OK : NF_ERR_CUDA;
}
