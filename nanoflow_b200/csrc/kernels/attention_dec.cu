// Decode attention (one query token per request, GQA) fed by a TMA producer warp: the form that is meant to
// share an SM with a GEMM CTA.
//
// The kernel in attention.cu gives each of its four warps a private cp.async ring that the warp fills
// itself: 32 copy instructions per lane and page, and at most 2-3 pages per warp in flight. With one
// such CTA per SM (all that fits beside a GEMM CTA) too few bytes are in flight and it runs at less than
// half of the memory bandwidth. Here one producer warp issues the copies: four TMA tile copies per page
// (K and V of one head, 8 KB, landing in the 128-byte-swizzled layout that ldmatrix reads without bank
// conflicts), into a ring of ST pages per consumer warp, completion through mbarriers. The four consumer
// warps spend their issue slots on ldmatrix / mma.sync / softmax only, and each owns whole work items
// (request x kv head): no cross-warp merge, no CTA-wide barrier in the steady state. Bytes in flight per
// CTA: 4 * ST * 8 KB (96 KB at ST = 3), independent of what the consumers are doing.
//
// Math per page is the one of attention.cu (the `group` query heads of a KV head are the rows of a
// 16-row mma.sync tile, online softmax in fp32, exp2 domain). head_dim 128, no split-KV: contexts that
// need splitting (few requests with long contexts) stay with attention.cu.
//
// Counterpart in the reference: BatchPrefillWithPagedKVCacheKernel_Small used for GQA decode with a
// bounded grid (gemv/include/attention/prefill.cuh:1376-1713), launched beside the GEMMs
// (pipeline/src/pipeline.cu:645-657).
#include "attn_mma.cuh"
#include "common.cuh"
#include "kernels.h"

namespace nf {
namespace {

constexpr int HD = 128;
constexpr int kConsumers = 4;
constexpr int kThreads = (kConsumers + 1) * 32;
constexpr int kPageBytes = kPage * HD * 2;        // one head's K (or V) page: 4 KB
constexpr int kStageBytes = 2 * kPageBytes;       // K + V

// byte offset of (token row, 16-byte chunk) inside a page stored as two [16 tok][64 hd] halves, 128-byte
// rows, chunk position XORed with the row (what TMA SWIZZLE_128B writes)
__device__ __forceinline__ uint32_t page_off(int row, int chunk) {
  return static_cast<uint32_t>((chunk >> 3) * 2048 + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

// S(16 x 16 tokens) += Q K^T over one page
__device__ __forceinline__ void qk_page(float (&s0)[4], float (&s1)[4], const uint32_t (&qa)[HD / 16][4],
                                        uint32_t k_base) {
  const int lane = threadIdx.x & 31;
  const int m = lane >> 3, r = lane & 7;
  const int tok = (m >> 1) * 8 + r;
#pragma unroll
  for (int ks = 0; ks < HD / 16; ++ks) {
    uint32_t b0, b1, b2, b3;
    ldsm_x4(k_base + page_off(tok, 2 * ks + (m & 1)), b0, b1, b2, b3);
    mma_bf16(s0, qa[ks], b0, b1);
    mma_bf16(s1, qa[ks], b2, b3);
  }
}
// O(16 x HD) += P(16 x 16 tokens) V over one page
__device__ __forceinline__ void pv_page(float (&o)[HD / 8][4], const uint32_t (&pa)[4], uint32_t v_base) {
  const int lane = threadIdx.x & 31;
  const int m = lane >> 3, r = lane & 7;
  const int tok = (m & 1) * 8 + r;
#pragma unroll
  for (int c = 0; c < HD / 8; c += 2) {
    uint32_t b0, b1, b2, b3;
    ldsm_x4_trans(v_base + page_off(tok, c + (m >> 1)), b0, b1, b2, b3);
    mma_bf16(o[c], pa, b0, b1);
    mma_bf16(o[c + 1], pa, b2, b3);
  }
}

template <int ST>
__global__ void __launch_bounds__(kThreads, 3)
attn_decode_tma_kernel(const __grid_constant__ CUtensorMap tmKV, nfk_attn_params p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sb = smem_u32(smem);
  constexpr int kRing = kConsumers * ST * kStageBytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kRing);      // [kConsumers][ST]
  uint64_t* empty = full + kConsumers * ST;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + kConsumers * ST);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if ((sb & 1023u) != 0u) {
    if (threadIdx.x == 0) report_status(p.status, NF_ST_BAD_INDEX);   // the swizzle assumes a 1024-aligned base
    return;
  }
  if (threadIdx.x == 0) {
    for (int i = 0; i < kConsumers * ST; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmKV);
  }
  __syncthreads();

  const int group = p.q_heads / p.kv_heads;
  const long long total = static_cast<long long>(p.req_count) * p.kv_heads;
  // work items are dealt to (CTA, consumer warp) slots round-robin; producer lane w and consumer warp w
  // walk the same list
  const long long slot0 = static_cast<long long>(blockIdx.x) * kConsumers;
  const long long stride = static_cast<long long>(gridDim.x) * kConsumers;

  if (warp == kConsumers) {
    // ------------------------------------------------------------------ producer: lane w feeds warp w
    if (lane < kConsumers) {
      const int w = lane;
      uint32_t cnt = 0;
      bool ok = true;
      for (long long item = slot0 + w; item < total && ok; item += stride) {
        const int kvh = static_cast<int>(item % p.kv_heads);
        const int req = p.req_begin + static_cast<int>(item / p.kv_heads);
        const int pg0 = p.kv_indptr[req];
        const int np = p.kv_indptr[req + 1] - pg0;
        int next_page = np > 0 ? p.kv_indices[pg0] : 0;
        for (int i = 0; i < np; ++i, ++cnt) {
          int page = next_page;
          if (i + 1 < np) next_page = p.kv_indices[pg0 + i + 1];     // in flight while this page is issued
          if (page < 0 || page >= p.num_pages) {
            report_status(p.status, NF_ST_BAD_INDEX);
            page = 0;
          }
          const int s = cnt % ST;
          uint64_t* fb = &full[w * ST + s];
          if (!mbar_wait(&empty[w * ST + s], ((cnt / ST) & 1) ^ 1) || *abort_flag) {
            report_status(p.status, NF_ST_TIMEOUT_SMEM_EMPTY);
            *abort_flag = 1;
            ok = false;
            break;
          }
          mbar_expect_tx(fb, kStageBytes);
          uint8_t* dst = smem + (w * ST + s) * kStageBytes;
          const int krow = ((page * 2) * p.kv_heads + kvh) * kPage;     // row of the [pages*2*kv_heads*16][128] view
          const int vrow = krow + p.kv_heads * kPage;
          tma_load_2d(dst, &tmKV, fb, 0, krow);
          tma_load_2d(dst + 2048, &tmKV, fb, 64, krow);
          tma_load_2d(dst + kPageBytes, &tmKV, fb, 0, vrow);
          tma_load_2d(dst + kPageBytes + 2048, &tmKV, fb, 64, vrow);
        }
      }
      // copies still in flight must land before the CTA gives its shared memory back
      const uint32_t back = cnt < static_cast<uint32_t>(ST) ? cnt : ST;
      for (uint32_t j = cnt - back; j < cnt; ++j) (void)mbar_wait(&full[w * ST + j % ST], (j / ST) & 1);
    }
    return;
  }

  // -------------------------------------------------------------------- consumers: one item per warp at a time
  const int w = warp;
  const __nv_bfloat16* qbase = reinterpret_cast<const __nv_bfloat16*>(p.q);
  __nv_bfloat16* outp = reinterpret_cast<__nv_bfloat16*>(p.out);
  const float scale = p.sm_scale * kLog2e;
  uint32_t cnt = 0;
  for (long long item = slot0 + w; item < total; item += stride) {
    const int kvh = static_cast<int>(item % p.kv_heads);
    const int req = p.req_begin + static_cast<int>(item / p.kv_heads);
    const int np = p.kv_indptr[req + 1] - p.kv_indptr[req];
    const int last_len = p.kv_last_page_len[req];
    const int tok = p.qo_indptr[req];
    uint32_t qa[HD / 16][4];
    load_q_frags<HD>(qa, [&](int r) -> const __nv_bfloat16* {
      return r < group ? qbase + (static_cast<long long>(tok) * p.q_heads + kvh * group + r) * HD : nullptr;
    });
    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    bool ok = true;
    for (int i = 0; i < np; ++i, ++cnt) {
      const int s = cnt % ST;
      const bool got = mbar_wait(&full[w * ST + s], (cnt / ST) & 1) && !*abort_flag;
      if (!__all_sync(0xffffffffu, got)) {     // the warp leaves as a whole: the MMAs below need all lanes
        if (lane == 0) report_status(p.status, NF_ST_TIMEOUT_SMEM_FULL);
        *abort_flag = 1;
        ok = false;
        break;
      }
      const uint32_t st = sb + (w * ST + s) * kStageBytes;
      float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
      qk_page(s0, s1, qa, st);
      const int valid = (i == np - 1) ? last_len : kPage;
      const int c0 = (lane & 3) * 2;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        s0[e] = (c0 + (e & 1) < valid) ? s0[e] * scale : -INFINITY;
        s1[e] = (8 + c0 + (e & 1) < valid) ? s1[e] * scale : -INFINITY;
      }
      const float mx0 = quad_max(fmaxf(fmaxf(s0[0], s0[1]), fmaxf(s1[0], s1[1])));
      const float mx1 = quad_max(fmaxf(fmaxf(s0[2], s0[3]), fmaxf(s1[2], s1[3])));
      const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
      const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;
      const float a0 = fast_exp2(m0 - ms0), a1 = fast_exp2(m1 - ms1);
      m0 = mn0;
      m1 = mn1;
      float pr[8];
      pr[0] = fast_exp2(s0[0] - ms0); pr[1] = fast_exp2(s0[1] - ms0);
      pr[2] = fast_exp2(s0[2] - ms1); pr[3] = fast_exp2(s0[3] - ms1);
      pr[4] = fast_exp2(s1[0] - ms0); pr[5] = fast_exp2(s1[1] - ms0);
      pr[6] = fast_exp2(s1[2] - ms1); pr[7] = fast_exp2(s1[3] - ms1);
      l0 = l0 * a0 + pr[0] + pr[1] + pr[4] + pr[5];
      l1 = l1 * a1 + pr[2] + pr[3] + pr[6] + pr[7];
#pragma unroll
      for (int c = 0; c < HD / 8; ++c) {
        o[c][0] *= a0; o[c][1] *= a0; o[c][2] *= a1; o[c][3] *= a1;
      }
      uint32_t pa[4];
      pa[0] = pack_bf16x2(pr[0], pr[1]);
      pa[1] = pack_bf16x2(pr[2], pr[3]);
      pa[2] = pack_bf16x2(pr[4], pr[5]);
      pa[3] = pack_bf16x2(pr[6], pr[7]);
      pv_page(o, pa, st + kPageBytes);
      __syncwarp();                                   // every lane is done reading the stage
      if (lane == 0) mbar_arrive(&empty[w * ST + s]);
    }
    if (!ok) return;
    l0 = quad_sum(l0);
    l1 = quad_sum(l1);
    const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
    const int r0 = lane >> 2, c0 = (lane & 3) * 2;
    if (r0 < group) {
      __nv_bfloat16* dst = outp + (static_cast<long long>(tok) * p.q_heads + kvh * group + r0) * HD;
#pragma unroll
      for (int c = 0; c < HD / 8; ++c)
        *reinterpret_cast<uint32_t*>(dst + c * 8 + c0) = pack_bf16x2(o[c][0] * inv0, o[c][1] * inv0);
    }
    if (r0 + 8 < group) {
      __nv_bfloat16* dst = outp + (static_cast<long long>(tok) * p.q_heads + kvh * group + r0 + 8) * HD;
#pragma unroll
      for (int c = 0; c < HD / 8; ++c)
        *reinterpret_cast<uint32_t*>(dst + c * 8 + c0) = pack_bf16x2(o[c][2] * inv1, o[c][3] * inv1);
    }
  }
}

template <int ST>
int launch_decode_tma(const nfk_attn_params* p, const CUtensorMap& tm, cudaStream_t stream) {
  constexpr int smem_bytes = kConsumers * ST * kStageBytes + 2 * kConsumers * ST * 8 + 64;
  static bool attr_dev[kMaxDevices] = {false};   // the attribute is per device
  bool& attr = attr_dev[device_slot()];
  if (!attr) {
    if (cudaFuncSetAttribute(attn_decode_tma_kernel<ST>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) !=
        cudaSuccess)
      return NF_ERR_CUDA;
    // beside a GEMM CTA the SM must keep its largest shared-memory split whichever kernel came first
    (void)cudaFuncSetAttribute(attn_decode_tma_kernel<ST>, cudaFuncAttributePreferredSharedMemoryCarveout,
                               cudaSharedmemCarveoutMaxShared);
    (void)cudaGetLastError();
    attr = true;
  }
  const long long total = static_cast<long long>(p->req_count) * p->kv_heads;
  const long long slots = (total + kConsumers - 1) / kConsumers;
  long long ctas = p->num_ctas > 0 ? p->num_ctas : 2LL * device_sm_count();
  if (ctas > slots) ctas = slots;
  attn_decode_tma_kernel<ST><<<static_cast<int>(ctas), kThreads, smem_bytes, stream>>>(tm, *p);
  return cudaGetLastError() == cudaSuccess ? NF_OK : NF_ERR_CUDA;
}

}  // namespace
}  // namespace nf

// Decode attention with a TMA producer warp (see the top of this file). Same contract as nfk_attn_decode
// without split-KV (chunk_pages must be 0) for head_dim 128; decode_stages = pages in flight per consumer
// warp: 2, 3 (0 means 3) or 4, i.e. 64 / 96 / 128 KB of shared memory per CTA.
extern "C" int nfk_attn_decode_tma(const nfk_attn_params* p, cudaStream_t stream) {
  using namespace nf;
  if (p == nullptr) return NF_ERR_BAD_ARG;
  if (!p->q || !p->out || !p->kv_pool || !p->qo_indptr || !p->kv_indptr || !p->kv_indices || !p->kv_last_page_len)
    return NF_ERR_BAD_ARG;
  if (p->kv_heads <= 0 || p->q_heads % p->kv_heads != 0 || p->num_pages <= 0) return NF_ERR_BAD_ARG;
  const int group = p->q_heads / p->kv_heads;
  if (p->head_dim != HD || p->page_size != kPage || group > 16 || (16 % group) != 0) return NF_ERR_UNSUPPORTED;
  if (p->chunk_pages != 0) {
    // split-KV iterations (few requests with long contexts) go to the kernel that has the merge pass
    nfk_attn_params q = *p;
    q.decode_stages = p->decode_stages == 2 ? 2 : 3;
    return nfk_attn_decode(&q, stream);
  }
  if (p->req_count == 0) return NF_OK;
  if (p->req_count < 0 || p->req_begin < 0) return NF_ERR_BAD_ARG;
  CUtensorMap tm;
  const int rc = make_tmap_bf16_2d(&tm, p->kv_pool, static_cast<uint64_t>(p->num_pages) * 2 * p->kv_heads * kPage, HD,
                                   HD, kPage, 64);
  if (rc != NF_OK) return rc;
  switch (p->decode_stages) {
    case 2: return launch_decode_tma<2>(p, tm, stream);
    case 0:
    case 3: return launch_decode_tma<3>(p, tm, stream);
    case 4: return launch_decode_tma<4>(p, tm, stream);
    default: return NF_ERR_BAD_ARG;
  }
}
