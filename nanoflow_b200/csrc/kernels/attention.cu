// Attention over the paged KV pool [pages][2][kv_heads][16][head_dim] (bf16, 16-token pages).
//
// nfk_attn_decode   one query token per request, GQA: the `group` query heads that share a KV head
//                   form the rows of a 16-row tensor-core tile. Persistent grid with a CTA budget;
//                   a work item is (request, kv head, kv chunk). The four warps of a CTA take
//                   alternate pages of the item, each with its own cp.async ring, and merge their
//                   softmax states in shared memory at the end. Optional split-KV writes per-chunk
//                   partials to a workspace that nfk_attn_decode's second launch merges.
// nfk_attn_prefill  causal, ragged query lengths (chunked prefill). A work item is (request, first
//                   token, token count <= 128/group) x kv head; 8 warps x 16 rows, K/V tiles of 64
//                   tokens double-buffered in shared memory and shared by all warps.
//
// Both are bandwidth-shaped flash-attention loops (online softmax in fp32, exp2 domain). The
// decode kernel is bound by HBM, so the tile math uses warp-level mma.sync, which is far from
// limiting at 8 FLOP per KV byte. Shared-memory rows are XOR-swizzled in 16-byte chunks so the
// ldmatrix reads are conflict free.
//
// Counterparts in the reference: the SM-limited persistent FlashInfer kernels
// BatchPrefillWithPagedKVCacheKernel_Small used for GQA decode (gemv/include/attention/prefill.cuh:1376-1713),
// BatchPrefillWithPagedKVCacheKernel (prefill.cuh:1066-1374), the partition-KV merge
// (gemv/include/attention/decode.cuh:827-872) and the wrappers in pipeline/include/gemvWrapper.cuh:140-237, :322-374.
#include "common.cuh"
#include "kernels.h"
#include "attn_decode_static.h"
#include "attn_mma.cuh"

#include <atomic>
#include <mutex>

namespace nf {
namespace {

// Shared-memory byte offset of (token row, 16-byte chunk) inside a [rows][HD] bf16 tile.
template <int HD>
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
  return static_cast<uint32_t>(row * (HD * 2) + ((chunk ^ (row & 7)) << 4));
}

// S(16 x 16 tokens) += Q K^T for one 16-token group starting at smem row `row0` of a K tile.
template <int HD>
__device__ __forceinline__ void qk_16tok(float (&s0)[4], float (&s1)[4],
                                         const uint32_t (&qa)[HD / 16][4], uint32_t k_base,
                                         int row0) {
  const int lane = threadIdx.x & 31;
  const int m = lane >> 3, r = lane & 7;
  const int tok = row0 + (m >> 1) * 8 + r;
#pragma unroll
  for (int ks = 0; ks < HD / 16; ++ks) {
    uint32_t b0, b1, b2, b3;
    ldsm_x4(k_base + tile_off<HD>(tok, 2 * ks + (m & 1)), b0, b1, b2, b3);
    mma_bf16(s0, qa[ks], b0, b1);
    mma_bf16(s1, qa[ks], b2, b3);
  }
}

// O(16 x HD) += P(16 x 16 tokens) V for the 16-token group at smem row `row0` of a V tile.
template <int HD>
__device__ __forceinline__ void pv_16tok(float (&o)[HD / 8][4], const uint32_t (&pa)[4],
                                         uint32_t v_base, int row0) {
  const int lane = threadIdx.x & 31;
  const int m = lane >> 3, r = lane & 7;
  const int tok = row0 + (m & 1) * 8 + r;
#pragma unroll
  for (int c = 0; c < HD / 8; c += 2) {
    uint32_t b0, b1, b2, b3;
    ldsm_x4_trans(v_base + tile_off<HD>(tok, c + (m >> 1)), b0, b1, b2, b3);
    mma_bf16(o[c], pa, b0, b1);
    mma_bf16(o[c + 1], pa, b2, b3);
  }
}

// ================================================================================================
// Decode
// ================================================================================================
constexpr int kDecThreads = 128;

// ST = pages in flight per warp (pipeline stages). 3 is the default (96 KB per CTA at head_dim 128, two
// CTAs per SM); 2 (64 KB) is for the case where a decode CTA shares an SM with a GEMM CTA and a
// collective's CTA (130 KB + 64 KB + the per-CTA reserve leave room, 130 KB + 96 KB do not).
template <int HD, int ST>
struct DecCfg {
  static constexpr int PAGE_BYTES = kPage * HD * 2;            // one head's K (or V) page
  static constexpr int STAGE_BYTES = 2 * PAGE_BYTES;           // K + V
  static constexpr int WARP_BYTES = ST * STAGE_BYTES;
  static constexpr int PIPE_BYTES = 4 * WARP_BYTES;
  static constexpr int MERGE_BYTES = 4 * (16 * HD * 4 + 16 * 2 * 4);
  static constexpr int SMEM_BYTES = PIPE_BYTES > MERGE_BYTES ? PIPE_BYTES : MERGE_BYTES;
};

// Work items are handed out through a counter: a CTA takes its first item by its index and every further
// one with an atomic increment, so CTAs that run slower (an SM shared with another kernel's CTA, a long
// context) take fewer items instead of holding up the launch. One counter pair per launch slot; launches
// cycle through the slots, and the last CTA of a launch to finish resets its slot.
constexpr int kDecodeCounterSlots = 64;
__device__ unsigned int g_decode_counters[kDecodeCounterSlots][2];

template <int HD, int ST>
__global__ void __launch_bounds__(kDecThreads, 3)
attn_decode_kernel(nfk_attn_params p, int slot) {
  using Cfg = DecCfg<HD, ST>;
  constexpr int kDecStages = ST;
  extern __shared__ __align__(128) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = p.q_heads / p.kv_heads;
  const int max_chunks = p.chunk_pages > 0 ? p.max_chunks : 1;
  const long long total = static_cast<long long>(p.req_count) * p.kv_heads * max_chunks;
  const __nv_bfloat16* qbase = reinterpret_cast<const __nv_bfloat16*>(p.q);
  const __nv_bfloat16* pool = reinterpret_cast<const __nv_bfloat16*>(p.kv_pool);
  __nv_bfloat16* outp = reinterpret_cast<__nv_bfloat16*>(p.out);
  const float scale = p.sm_scale * kLog2e;
  const uint32_t warp_smem = smem_u32(smem) + warp * Cfg::WARP_BYTES;

  unsigned int* counters = g_decode_counters[slot];
  long long item = blockIdx.x;
  while (item < total) {
    // the index of the item after this one is fetched now (thread 0 keeps it) and handed to the CTA through
    // the first word of the pipeline buffers once this item no longer needs them
    long long fetched = 0;
    if (threadIdx.x == 0) fetched = static_cast<long long>(gridDim.x) + atomicAdd(&counters[0], 1u);
    do {
    const int chunk = static_cast<int>(item % max_chunks);
    const int kvh = static_cast<int>((item / max_chunks) % p.kv_heads);
    const int bl = static_cast<int>(item / (static_cast<long long>(max_chunks) * p.kv_heads));
    const int req = p.req_begin + bl;
    const int pg0 = p.kv_indptr[req];
    const int np = p.kv_indptr[req + 1] - pg0;
    const int last_len = p.kv_last_page_len[req];
    int c_begin = 0, c_end = np, n_chunks = 1;
    if (p.chunk_pages > 0) {
      // A context longer than chunk_pages * max_chunks pages still has only max_chunks work items:
      // the last one takes all remaining pages, and the merge below counts the same number of chunks.
      c_begin = chunk * p.chunk_pages;
      c_end = (chunk == max_chunks - 1) ? np : min(np, c_begin + p.chunk_pages);
      n_chunks = min(max_chunks, (np + p.chunk_pages - 1) / p.chunk_pages);
    }
    if (c_begin >= c_end) break;  // uniform across the CTA: on to the next item
    const int tok = p.qo_indptr[req];

    uint32_t qa[HD / 16][4];
    load_q_frags<HD>(qa, [&](int r) -> const __nv_bfloat16* {
      return r < group ? qbase + (static_cast<long long>(tok) * p.q_heads + kvh * group + r) * HD
                       : nullptr;
    });

    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    // This warp's pages: c_begin + warp, + 4, + 8, ...
    const int my_n = (c_end - c_begin - warp + 3) / 4;  // may be <= 0
    auto issue = [&](int i) {
      if (i < my_n) {
        const int pslot = c_begin + warp + 4 * i;
        int page = p.kv_indices[pg0 + pslot];
        if (page < 0 || page >= p.num_pages) {
          if (lane == 0) report_status(p.status, NF_ST_BAD_INDEX);
          page = 0;
        }
        const __nv_bfloat16* kp =
            pool + ((static_cast<long long>(page) * 2) * p.kv_heads + kvh) * (kPage * HD);
        const __nv_bfloat16* vp = kp + static_cast<long long>(p.kv_heads) * (kPage * HD);
        const uint32_t st = warp_smem + (i % kDecStages) * Cfg::STAGE_BYTES;
#pragma unroll
        for (int j = 0; j < (kPage * HD / 8) / 32; ++j) {
          const int idx = lane + 32 * j;
          const int row = idx / (HD / 8), ch = idx % (HD / 8);
          cp_async16(st + tile_off<HD>(row, ch), kp + idx * 8);
          cp_async16(st + Cfg::PAGE_BYTES + tile_off<HD>(row, ch), vp + idx * 8);
        }
      }
      cp_async_commit();
    };
#pragma unroll
    for (int s = 0; s < kDecStages - 1; ++s) issue(s);

    for (int i = 0; i < my_n; ++i) {
      cp_async_wait<kDecStages - 2>();
      __syncwarp();
      const uint32_t st = warp_smem + (i % kDecStages) * Cfg::STAGE_BYTES;
      float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
      qk_16tok<HD>(s0, s1, qa, st, 0);
      const int pslot = c_begin + warp + 4 * i;
      const int valid = (pslot == np - 1) ? last_len : kPage;
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
      pv_16tok<HD>(o, pa, st + Cfg::PAGE_BYTES, 0);
      __syncwarp();
      issue(i + kDecStages - 1);
    }
    cp_async_wait<0>();
    l0 = quad_sum(l0);
    l1 = quad_sum(l1);

    // ---- merge the four warps through shared memory (reuses the pipeline buffers) ----
    __syncthreads();
    float* mo = reinterpret_cast<float*>(smem);              // [4][16][HD]
    float* mml = mo + 4 * 16 * HD;                           // [4][16][2] (m, l)
    {
      const int r0 = lane >> 2, c0 = (lane & 3) * 2;
      float* wo = mo + warp * 16 * HD;
#pragma unroll
      for (int c = 0; c < HD / 8; ++c) {
        *reinterpret_cast<float2*>(wo + r0 * HD + c * 8 + c0) = make_float2(o[c][0], o[c][1]);
        *reinterpret_cast<float2*>(wo + (r0 + 8) * HD + c * 8 + c0) = make_float2(o[c][2], o[c][3]);
      }
      if ((lane & 3) == 0) {
        mml[(warp * 16 + r0) * 2] = m0;
        mml[(warp * 16 + r0) * 2 + 1] = l0;
        mml[(warp * 16 + r0 + 8) * 2] = m1;
        mml[(warp * 16 + r0 + 8) * 2 + 1] = l1;
      }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < group * (HD / 2); idx += kDecThreads) {
      const int r = idx / (HD / 2), c = (idx % (HD / 2)) * 2;
      float mm = -INFINITY;
#pragma unroll
      for (int w = 0; w < 4; ++w) mm = fmaxf(mm, mml[(w * 16 + r) * 2]);
      const float msafe = mm == -INFINITY ? 0.f : mm;
      float L = 0.f, x = 0.f, y = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float sc = fast_exp2(mml[(w * 16 + r) * 2] - msafe);
        L += mml[(w * 16 + r) * 2 + 1] * sc;
        const float2 v = *reinterpret_cast<const float2*>(mo + (w * 16 + r) * HD + c);
        x += v.x * sc;
        y += v.y * sc;
      }
      const float inv = L > 0.f ? 1.f / L : 0.f;
      const int head = kvh * group + r;
      if (n_chunks == 1) {
        *reinterpret_cast<uint32_t*>(outp + (static_cast<long long>(tok) * p.q_heads + head) * HD + c) =
            pack_bf16x2(x * inv, y * inv);
      } else {
        float* ws = p.workspace +
                    ((static_cast<long long>(bl) * p.q_heads + head) * max_chunks + chunk) * (HD + 2);
        *reinterpret_cast<float2*>(ws + c) = make_float2(x * inv, y * inv);
        if (c == 0) ws[HD] = L > 0.f ? mm + log2f(L) : -INFINITY;
      }
    }
    } while (false);
    __syncthreads();  // every warp is done with the pipeline buffers and the merge area
    if (threadIdx.x == 0) *reinterpret_cast<long long*>(smem) = fetched;
    __syncthreads();
    item = *reinterpret_cast<const long long*>(smem);
    __syncthreads();  // ... before the next item's loads overwrite the word
  }
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(&counters[1], 1u);
    if (prev == gridDim.x - 1) {      // every CTA has taken its last item: the slot is free again
      counters[0] = 0;
      counters[1] = 0;
    }
  }
}

template <int HD>
__global__ void attn_decode_merge_kernel(nfk_attn_params p) {
  const int bl = blockIdx.x / p.q_heads, head = blockIdx.x % p.q_heads;
  const int req = p.req_begin + bl;
  const int np = p.kv_indptr[req + 1] - p.kv_indptr[req];
  const int n_chunks = min(p.max_chunks, (np + p.chunk_pages - 1) / p.chunk_pages);   // as in the decode kernel
  if (n_chunks <= 1) return;  // the decode kernel already wrote the final rows
  const float* ws = p.workspace + (static_cast<long long>(bl) * p.q_heads + head) * p.max_chunks * (HD + 2);
  float mm = -INFINITY;
  for (int c = 0; c < n_chunks; ++c) mm = fmaxf(mm, ws[c * (HD + 2) + HD]);
  const float msafe = mm == -INFINITY ? 0.f : mm;
  const int tok = p.qo_indptr[req];
  __nv_bfloat16* outp = reinterpret_cast<__nv_bfloat16*>(p.out);
  for (int d = threadIdx.x; d < HD; d += blockDim.x) {
    float acc = 0.f, W = 0.f;
    for (int c = 0; c < n_chunks; ++c) {
      const float w = exp2f(ws[c * (HD + 2) + HD] - msafe);
      W += w;
      acc += w * ws[c * (HD + 2) + d];
    }
    outp[(static_cast<long long>(tok) * p.q_heads + head) * HD + d] =
        __float2bfloat16(W > 0.f ? acc / W : 0.f);
  }
}

// ================================================================================================
// Prefill (causal, ragged)
// ================================================================================================
constexpr int kPreThreads = 256;
constexpr int kPreTile = 64;  // kv tokens per tile

template <int HD>
struct PreCfg {
  static constexpr int TILE_BYTES = kPreTile * HD * 2;
  static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  static constexpr int SMEM_BYTES = 2 * STAGE_BYTES;
};

template <int HD>
__global__ void __launch_bounds__(kPreThreads, 1)
attn_prefill_kernel(nfk_attn_params p) {
  using Cfg = PreCfg<HD>;
  extern __shared__ __align__(128) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = p.q_heads / p.kv_heads;
  const long long total = static_cast<long long>(p.num_items) * p.kv_heads;
  const __nv_bfloat16* qbase = reinterpret_cast<const __nv_bfloat16*>(p.q);
  const __nv_bfloat16* pool = reinterpret_cast<const __nv_bfloat16*>(p.kv_pool);
  __nv_bfloat16* outp = reinterpret_cast<__nv_bfloat16*>(p.out);
  const float scale = p.sm_scale * kLog2e;
  const uint32_t smem_base = smem_u32(smem);

  for (long long w = blockIdx.x; w < total; w += gridDim.x) {
    const int item = static_cast<int>(w / p.kv_heads);
    const int kvh = static_cast<int>(w % p.kv_heads);
    const int req = p.items[item * 3 + 0];
    const int tok0 = p.items[item * 3 + 1];
    const int ntok = p.items[item * 3 + 2];
    const int pg0 = p.kv_indptr[req];
    const int np = p.kv_indptr[req + 1] - pg0;
    const int kv_len = (np - 1) * kPage + p.kv_last_page_len[req];
    const int q_end = p.qo_indptr[req + 1];
    // absolute position of global token t of this request: kv_len - (q_end - t)
    const int kv_hi = kv_len - (q_end - (tok0 + ntok - 1)) + 1;  // keys visible to the last row
    if (ntok <= 0 || np <= 0 || kv_hi <= 0) continue;
    const int n_tiles = (kv_hi + kPreTile - 1) / kPreTile;

    // rows of this warp: r = warp*16 + i -> token r / group, head r % group
    const int rbase = warp * 16;
    auto row_tok = [&](int i) { return (rbase + i) / group; };
    auto row_head = [&](int i) { return (rbase + i) % group; };
    uint32_t qa[HD / 16][4];
    load_q_frags<HD>(qa, [&](int i) -> const __nv_bfloat16* {
      const int tl = row_tok(i);
      return tl < ntok ? qbase + (static_cast<long long>(tok0 + tl) * p.q_heads + kvh * group +
                                  row_head(i)) * HD
                       : nullptr;
    });
    const int i0 = lane >> 2, i1 = i0 + 8;
    const int pos0 = row_tok(i0) < ntok ? kv_len - (q_end - (tok0 + row_tok(i0))) : -1;
    const int pos1 = row_tok(i1) < ntok ? kv_len - (q_end - (tok0 + row_tok(i1))) : -1;

    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    auto issue = [&](int t) {
      if (t < n_tiles) {
        const uint32_t st = smem_base + (t & 1) * Cfg::STAGE_BYTES;
        constexpr int CHUNKS = kPreTile * HD / 8;  // 16-byte chunks per K (or V) tile
#pragma unroll
        for (int j = 0; j < CHUNKS / kPreThreads; ++j) {
          const int idx = threadIdx.x + kPreThreads * j;
          const int row = idx / (HD / 8), ch = idx % (HD / 8);
          int pslot = t * (kPreTile / kPage) + row / kPage;
          if (pslot >= np) pslot = 0;  // past the sequence: re-read a valid page, masked below
          int page = p.kv_indices[pg0 + pslot];
          if (page < 0 || page >= p.num_pages) {
            report_status(p.status, NF_ST_BAD_INDEX);
            page = 0;
          }
          const __nv_bfloat16* kp = pool +
              ((static_cast<long long>(page) * 2) * p.kv_heads + kvh) * (kPage * HD) +
              (row % kPage) * HD + ch * 8;
          cp_async16(st + tile_off<HD>(row, ch), kp);
          cp_async16(st + Cfg::TILE_BYTES + tile_off<HD>(row, ch),
                     kp + static_cast<long long>(p.kv_heads) * (kPage * HD));
        }
      }
      cp_async_commit();
    };

    issue(0);
    for (int t = 0; t < n_tiles; ++t) {
      issue(t + 1);
      cp_async_wait<1>();
      __syncthreads();
      const uint32_t st = smem_base + (t & 1) * Cfg::STAGE_BYTES;
      float s[kPreTile / 8][4];
#pragma unroll
      for (int n = 0; n < kPreTile / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
      for (int g = 0; g < kPreTile / 16; ++g) qk_16tok<HD>(s[2 * g], s[2 * g + 1], qa, st, g * 16);
      const int cbase = t * kPreTile + (lane & 3) * 2;
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int n = 0; n < kPreTile / 8; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int col = cbase + n * 8 + (e & 1);
          const int lim = (e < 2) ? pos0 : pos1;
          s[n][e] = (col <= lim) ? s[n][e] * scale : -INFINITY;
        }
        mx0 = fmaxf(mx0, fmaxf(s[n][0], s[n][1]));
        mx1 = fmaxf(mx1, fmaxf(s[n][2], s[n][3]));
      }
      mx0 = quad_max(mx0);
      mx1 = quad_max(mx1);
      const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
      const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;
      const float a0 = fast_exp2(m0 - ms0), a1 = fast_exp2(m1 - ms1);
      m0 = mn0;
      m1 = mn1;
      float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
      for (int n = 0; n < kPreTile / 8; ++n) {
        s[n][0] = fast_exp2(s[n][0] - ms0);
        s[n][1] = fast_exp2(s[n][1] - ms0);
        s[n][2] = fast_exp2(s[n][2] - ms1);
        s[n][3] = fast_exp2(s[n][3] - ms1);
        rs0 += s[n][0] + s[n][1];
        rs1 += s[n][2] + s[n][3];
      }
      l0 = l0 * a0 + rs0;
      l1 = l1 * a1 + rs1;
#pragma unroll
      for (int c = 0; c < HD / 8; ++c) {
        o[c][0] *= a0; o[c][1] *= a0; o[c][2] *= a1; o[c][3] *= a1;
      }
#pragma unroll
      for (int g = 0; g < kPreTile / 16; ++g) {
        uint32_t pa[4];
        pa[0] = pack_bf16x2(s[2 * g][0], s[2 * g][1]);
        pa[1] = pack_bf16x2(s[2 * g][2], s[2 * g][3]);
        pa[2] = pack_bf16x2(s[2 * g + 1][0], s[2 * g + 1][1]);
        pa[3] = pack_bf16x2(s[2 * g + 1][2], s[2 * g + 1][3]);
        pv_16tok<HD>(o, pa, st + Cfg::TILE_BYTES, g * 16);
      }
      __syncthreads();  // all warps done with this stage before it is refilled
    }
    cp_async_wait<0>();
    l0 = quad_sum(l0);
    l1 = quad_sum(l1);
    const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
    const int c0 = (lane & 3) * 2;
    if (row_tok(i0) < ntok) {
      __nv_bfloat16* dst = outp + (static_cast<long long>(tok0 + row_tok(i0)) * p.q_heads +
                                   kvh * group + row_head(i0)) * HD;
#pragma unroll
      for (int c = 0; c < HD / 8; ++c)
        *reinterpret_cast<uint32_t*>(dst + c * 8 + c0) = pack_bf16x2(o[c][0] * inv0, o[c][1] * inv0);
    }
    if (row_tok(i1) < ntok) {
      __nv_bfloat16* dst = outp + (static_cast<long long>(tok0 + row_tok(i1)) * p.q_heads +
                                   kvh * group + row_head(i1)) * HD;
#pragma unroll
      for (int c = 0; c < HD / 8; ++c)
        *reinterpret_cast<uint32_t*>(dst + c * 8 + c0) = pack_bf16x2(o[c][2] * inv1, o[c][3] * inv1);
    }
  }
}

inline int sm_count_attn() { return device_sm_count(); }

int check_common(const nfk_attn_params* p) {
  if (p == nullptr) return NF_ERR_BAD_ARG;
  if (!p->q || !p->out || !p->kv_pool || !p->qo_indptr || !p->kv_indptr || !p->kv_indices ||
      !p->kv_last_page_len)
    return NF_ERR_BAD_ARG;
  if (p->kv_heads <= 0 || p->q_heads % p->kv_heads != 0) return NF_ERR_BAD_ARG;
  const int group = p->q_heads / p->kv_heads;
  if (group > 16 || (16 % group) != 0) return NF_ERR_UNSUPPORTED;
  if (p->page_size != kPage) return NF_ERR_UNSUPPORTED;
  if (p->head_dim != 128 && p->head_dim != 64) return NF_ERR_UNSUPPORTED;
  return NF_OK;
}

template <int HD, int ST>
int launch_decode_st(const nfk_attn_params* p, cudaStream_t stream) {
  using Cfg = DecCfg<HD, ST>;
  static bool attr_dev[kMaxDevices] = {false};   // the attribute is per device
  bool& attr = attr_dev[device_slot()];
  if (!attr) {
    if (cudaFuncSetAttribute(attn_decode_kernel<HD, ST>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Cfg::SMEM_BYTES) != cudaSuccess)
      return NF_ERR_CUDA;
    attr = true;
  }
  const int max_chunks = p->chunk_pages > 0 ? p->max_chunks : 1;
  const long long total = static_cast<long long>(p->req_count) * p->kv_heads * max_chunks;
  long long ctas = p->num_ctas > 0 ? p->num_ctas : 2LL * sm_count_attn();
  if (ctas > total) ctas = total;
  static std::atomic<unsigned int> launch_seq{0};
  const int slot = static_cast<int>(launch_seq.fetch_add(1u) % kDecodeCounterSlots);
  attn_decode_kernel<HD, ST><<<static_cast<int>(ctas), kDecThreads, Cfg::SMEM_BYTES, stream>>>(*p, slot);
  if (cudaGetLastError() != cudaSuccess) return NF_ERR_CUDA;
  if (p->chunk_pages > 0 && max_chunks > 1) {
    attn_decode_merge_kernel<HD><<<p->req_count * p->q_heads, HD, 0, stream>>>(*p);
    if (cudaGetLastError() != cudaSuccess) return NF_ERR_CUDA;
  }
  return NF_OK;
}

template <int HD>
int launch_decode(const nfk_attn_params* p, cudaStream_t stream) {
  return p->decode_stages == 2 ? launch_decode_st<HD, 2>(p, stream) : launch_decode_st<HD, 3>(p, stream);
}

template <int HD>
int launch_prefill(const nfk_attn_params* p, cudaStream_t stream) {
  using Cfg = PreCfg<HD>;
  static bool attr_dev[kMaxDevices] = {false};   // the attribute is per device
  bool& attr = attr_dev[device_slot()];
  if (!attr) {
    if (cudaFuncSetAttribute(attn_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Cfg::SMEM_BYTES) != cudaSuccess)
      return NF_ERR_CUDA;
    attr = true;
  }
  const long long total = static_cast<long long>(p->num_items) * p->kv_heads;
  long long ctas = p->num_ctas > 0 ? p->num_ctas : sm_count_attn();
  if (ctas > total) ctas = total;
  attn_prefill_kernel<HD><<<static_cast<int>(ctas), kPreThreads, Cfg::SMEM_BYTES, stream>>>(*p);
  return cudaGetLastError() == cudaSuccess ? NF_OK : NF_ERR_CUDA;
}

}  // namespace
}  // namespace nf

extern "C" int nfk_attn_decode(const nfk_attn_params* p, cudaStream_t stream) {
  using namespace nf;
  const int rc = check_common(p);
  if (rc != NF_OK) return rc;
  if (p->req_count == 0) return NF_OK;
  if (p->req_count < 0 || p->req_begin < 0) return NF_ERR_BAD_ARG;
  if (p->chunk_pages < 0 || (p->chunk_pages > 0 && (p->max_chunks < 1 || p->workspace == nullptr)))
    return NF_ERR_BAD_ARG;
  if (p->decode_stages != 0 && p->decode_stages != 2 && p->decode_stages != 3) return NF_ERR_BAD_ARG;
  return p->head_dim == 128 ? launch_decode<128>(p, stream) : launch_decode<64>(p, stream);
}

// ------------------------------------------------------------------------------------------------
// Split-KV decode without any allocation: the per-chunk partial results live in a fixed array that
// is part of the library image instead of a caller-provided workspace.
// ------------------------------------------------------------------------------------------------
static __device__ __align__(256) float g_decode_static_scratch[NFK_ATTN_DECODE_STATIC_SCRATCH_FLOATS];

namespace nf {
namespace {
float* g_static_scratch_ptr[kMaxDevices] = {nullptr};

// Device address of the scratch array on the current device. In host code the array's name is only
// a handle for the runtime, never an address a kernel could use; the address has to be asked for,
// once per device, with that device current.
int static_scratch_for_current_device(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return NF_ERR_CUDA;
  // first calls from several host threads: one of them asks, the others wait for its answer
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  if (g_static_scratch_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_decode_static_scratch) != cudaSuccess || ptr == nullptr)
      return NF_ERR_CUDA;
    g_static_scratch_ptr[dev] = static_cast<float*>(ptr);
  }
  *out = g_static_scratch_ptr[dev];
  return NF_OK;
}
}  // namespace
}  // namespace nf

extern "C" int nfk_attn_decode_static(const nfk_attn_params* p, cudaStream_t stream) {
  using namespace nf;
  const int rc = check_common(p);
  if (rc != NF_OK) return rc;
  if (p->req_count == 0) return NF_OK;
  if (p->req_count < 0 || p->req_begin < 0 || p->chunk_pages < 0) return NF_ERR_BAD_ARG;
  if (p->decode_stages != 0 && p->decode_stages != 2 && p->decode_stages != 3) return NF_ERR_BAD_ARG;
  nfk_attn_params q = *p;
  q.workspace = nullptr;
  if (q.chunk_pages > 0) {
    if (q.max_chunks < 1) return NF_ERR_BAD_ARG;
    const long long need = static_cast<long long>(q.req_count) * q.q_heads * q.max_chunks * (q.head_dim + 2);
    if (need > NFK_ATTN_DECODE_STATIC_SCRATCH_FLOATS) return NF_ERR_BAD_ARG;   // beyond the fixed scratch
    float* scratch = nullptr;
    const int rs = static_scratch_for_current_device(&scratch);
    if (rs != NF_OK) return rs;
    q.workspace = scratch;
  }
  return q.head_dim == 128 ? launch_decode<128>(&q, stream) : launch_decode<64>(&q, stream);
}

extern "C" int nfk_attn_prefill(const nfk_attn_params* p, cudaStream_t stream) {
  using namespace nf;
  const int rc = check_common(p);
  if (rc != NF_OK) return rc;
  if (p->num_items == 0) return NF_OK;
  if (p->num_items < 0 || p->items == nullptr) return NF_ERR_BAD_ARG;
  return p->head_dim == 128 ? launch_prefill<128>(p, stream) : launch_prefill<64>(p, stream);
}
