// Chunked-prefill attention on the 5th-generation tensor cores (head_dim 128), warp-specialised.
//
// A work item is (request, first token, token count <= 128/group) x kv head, as in nfk_attn_prefill: the
// item's query rows r = token * group + head fill one 128-row MMA tile, and the item walks its keys in
// tiles of 64 tokens. Three roles share a 192-thread CTA and meet only through mbarriers:
//
//   warp 4, one thread   loads: TMA copies (no multicast) of the Q rows and of whole K / V pages from the
//                        paged pool into 128B-swizzled shared memory, two K and two V tiles in flight;
//                        the page ids of the next tile are fetched while the current one is issued
//   warp 5, one thread   tcgen05.mma: S(t+1) = Q K(t+1)^T is issued before P(t) is waited for, into the
//                        other of two S accumulators in TMEM, so the tensor cores work on the next tile's
//                        scores while the softmax warps are still busy with this tile; then
//                        O += P(t) V(t) with P read from TMEM (A operand in tensor memory) and V read
//                        token-major from shared memory (MN-major B operand: no transpose pass)
//   warps 0-3            softmax: one thread per query row reads its 64 scores from TMEM, keeps the
//                        running maximum and sum, and writes P (bf16, two per column) back over the first 32
//                        columns of the S accumulator it came from: P never passes through shared memory
//
// S(t+2) goes into the accumulator that held S(t) / P(t), so the MMA thread issues it only once
// O += P(t) V(t) has completed (products into different accumulators are not ordered against each other's
// operand reads); S(t+2) is needed a whole softmax pass later, so that wait is off the critical path.
//
// O stays in TMEM for the whole item: P is taken relative to a reference maximum that only moves (and O
// is rescaled in TMEM) when a row's maximum outgrows it by more than 2^8. Two CTAs fit an SM (97 KB of
// shared memory, 256 TMEM columns each). Every wait is bounded; a wait that runs out sets the status
// word and all roles leave through the common exit, which frees TMEM.
//
// Takes the place of the reference's FlashInfer BatchPrefillWithPagedKVCacheKernel
// (gemv/include/attention/prefill.cuh:1066-1374, mma.sync m16n16k16 + ldmatrix on sm_80).
#include "common.cuh"
#include "kernels.h"

namespace nf {
namespace {

constexpr int HD = 128;
constexpr int kPage = 16;
constexpr int kTile = 64;             // kv tokens per tile
constexpr int kThreads = 192;         // warps 0-3 softmax (TMEM lane quarter = warp index), 4 loads, 5 MMA
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleGap = 8.0f;   // log2 of how far a row maximum may outgrow its reference

// shared-memory map (bytes from the 1024-aligned base); every operand region is 1024-aligned
constexpr int Q_OFF = 0;                       // 2 halves x [128 rows][64 hd]                 32 KB
constexpr int K_OFF = 32768;                   // 2 stages x 2 halves x [64 tok][64 hd]        32 KB
constexpr int V_OFF = K_OFF + 32768;           // 2 stages x 2 halves x [64 tok][64 hd]        32 KB
constexpr int BAR_OFF = V_OFF + 32768;
constexpr int kSmemBytes = BAR_OFF + 256;
constexpr int kStageBytes = 16384;             // one K (or V) tile
constexpr int kHalfBytes = 8192;               // [64 tok][64 hd]

enum Bar : int {
  Q_FULL = 0, Q_EMPTY, K_FULL0, K_FULL1, K_EMPTY0, K_EMPTY1, V_FULL0, V_FULL1, V_EMPTY0, V_EMPTY1,
  S_FULL0, S_FULL1, P_FULL0, P_FULL1, PV_DONE0, PV_DONE1, O_FREE, NUM_BARS
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// Shared-memory descriptor of an MN-major operand in the 128-byte swizzle: 64 elements along M/N are
// contiguous (one 128-byte row per k index), `lbo` bytes lead to the next 64 elements along M/N, `sbo`
// bytes to the next group of eight k indices.
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>((lbo >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>((sbo >> 4) & 0x3FFF) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
constexpr uint32_t kIdescBMnMajor = 1u << 16;

struct Item {
  int req, tok0, ntok, kvh, pg0, np, kv_len, q_end, n_tiles;
  bool valid;
};
__device__ __forceinline__ Item read_item(const nfk_attn_params& p, long long w) {
  Item it;
  const int item = static_cast<int>(w / p.kv_heads);
  it.kvh = static_cast<int>(w % p.kv_heads);
  it.req = p.items[item * 3 + 0];
  it.tok0 = p.items[item * 3 + 1];
  it.ntok = p.items[item * 3 + 2];
  it.pg0 = p.kv_indptr[it.req];
  it.np = p.kv_indptr[it.req + 1] - it.pg0;
  it.kv_len = (it.np - 1) * kPage + p.kv_last_page_len[it.req];
  it.q_end = p.qo_indptr[it.req + 1];
  // absolute position of global token t of this request: kv_len - (q_end - t)
  const int kv_hi = it.kv_len - (it.q_end - (it.tok0 + it.ntok - 1)) + 1;   // keys visible to the last row
  it.valid = it.ntok > 0 && it.np > 0 && kv_hi > 0;
  it.n_tiles = it.valid ? (kv_hi + kTile - 1) / kTile : 0;
  return it;
}

__global__ void __launch_bounds__(kThreads, 2)
attn_prefill_ws_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmKV,
                       nfk_attn_params p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sb = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + BAR_OFF);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NUM_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if ((sb & 1023u) != 0u) {
    // the operand layouts assume a 1024-aligned base; report instead of computing garbage
    if (threadIdx.x == 0) report_status(p.status, NF_ST_BAD_INDEX);
    return;
  }

  if (threadIdx.x == 0) {
    for (int b = 0; b < NUM_BARS; ++b) {
      const bool warps4 = b == P_FULL0 || b == P_FULL1 || b == O_FREE;
      mbar_init(&bars[b], warps4 ? 4 : 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmKV);
  }
  // Q rows past an item's last token are never loaded; start them (and everything else) from zero so
  // that what the tensor cores read there is always finite
  for (int i = threadIdx.x; i < BAR_OFF / 16; i += kThreads) st_shared_v4(sb + i * 16, 0u, 0u, 0u, 0u);
  fence_proxy_async_smem();
  if (warp == 5) {
    tmem_alloc(tmem_slot, 256);   // S0: columns [0,64), S1: [64,128), O: [128,256)
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  const int group = p.q_heads / p.kv_heads;
  const long long total = static_cast<long long>(p.num_items) * p.kv_heads;
  auto fail = [&](unsigned int code) {
    report_status(p.status, code);
    *abort_flag = 1;
  };

  if (warp == 4) {
    // ------------------------------------------------------------------ loads
    if (lane == 0) {
      uint32_t g = 0, n_item = 0;          // tiles / items issued so far by this CTA
      uint32_t issued[NUM_BARS];           // per "full" barrier: loads issued on it
      for (int b = 0; b < NUM_BARS; ++b) issued[b] = 0;
      bool ok = true;
      for (long long w = blockIdx.x; w < total && ok; w += gridDim.x) {
        const Item it = read_item(p, w);
        if (!it.valid) continue;
        if (!mbar_wait(&bars[Q_EMPTY], (n_item & 1) ^ 1) || *abort_flag) { fail(NF_ST_TIMEOUT_SMEM_EMPTY); break; }
        mbar_expect_tx(&bars[Q_FULL], static_cast<uint32_t>(it.ntok * group) * HD * 2);
        for (int tl = 0; tl < it.ntok; ++tl) {
          const int grow = (it.tok0 + tl) * p.q_heads + it.kvh * group;     // row of the [T*q_heads][128] view
          tma_load_2d(smem + Q_OFF + tl * group * 128, &tmQ, &bars[Q_FULL], 0, grow);
          tma_load_2d(smem + Q_OFF + 16384 + tl * group * 128, &tmQ, &bars[Q_FULL], 64, grow);
        }
        ++issued[Q_FULL];
        ++n_item;
        int pages[4];
        auto fetch_pages = [&](int t) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            int pslot = t * (kTile / kPage) + j;
            if (pslot >= it.np) pslot = 0;      // past the sequence: a valid page, masked by position
            int page = p.kv_indices[it.pg0 + pslot];
            if (page < 0 || page >= p.num_pages) {
              report_status(p.status, NF_ST_BAD_INDEX);
              page = 0;
            }
            pages[j] = page;
          }
        };
        fetch_pages(0);
        for (int t = 0; t < it.n_tiles; ++t, ++g) {
          const int s = g & 1;
          const uint32_t ph = ((g >> 1) & 1) ^ 1;
          int cur[4] = {pages[0], pages[1], pages[2], pages[3]};
          if (t + 1 < it.n_tiles) fetch_pages(t + 1);     // in flight while this tile's copies are issued
          if (!mbar_wait(&bars[K_EMPTY0 + s], ph) || *abort_flag) { fail(NF_ST_TIMEOUT_SMEM_EMPTY); ok = false; break; }
          mbar_expect_tx(&bars[K_FULL0 + s], kStageBytes);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int row0 = ((cur[j] * 2) * p.kv_heads + it.kvh) * kPage;   // of the [pages*2*kv_heads*16][128] view
            uint8_t* dst = smem + K_OFF + s * kStageBytes + j * 2048;
            tma_load_2d(dst, &tmKV, &bars[K_FULL0 + s], 0, row0);
            tma_load_2d(dst + kHalfBytes, &tmKV, &bars[K_FULL0 + s], 64, row0);
          }
          ++issued[K_FULL0 + s];
          if (!mbar_wait(&bars[V_EMPTY0 + s], ph) || *abort_flag) { fail(NF_ST_TIMEOUT_SMEM_EMPTY); ok = false; break; }
          mbar_expect_tx(&bars[V_FULL0 + s], kStageBytes);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int row0 = ((cur[j] * 2 + 1) * p.kv_heads + it.kvh) * kPage;
            uint8_t* dst = smem + V_OFF + s * kStageBytes + j * 2048;
            tma_load_2d(dst, &tmKV, &bars[V_FULL0 + s], 0, row0);
            tma_load_2d(dst + kHalfBytes, &tmKV, &bars[V_FULL0 + s], 64, row0);
          }
          ++issued[V_FULL0 + s];
        }
      }
      // copies still in flight must have landed before the CTA gives its shared memory back
      const int fulls[5] = {Q_FULL, K_FULL0, K_FULL1, V_FULL0, V_FULL1};
      for (int i = 0; i < 5; ++i) {
        const int b = fulls[i];
        if (issued[b] > 0) (void)mbar_wait(&bars[b], (issued[b] - 1) & 1);
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issue
    if (lane == 0) {
      const uint32_t idesc_s = umma_idesc_bf16(128, kTile);
      const uint32_t idesc_o = umma_idesc_bf16(128, HD) | kIdescBMnMajor;
      uint32_t g = 0, n_item = 0;
      // `pv_issued`: PV products issued so far by this CTA. The S accumulator that S(gt) goes into held P(gt-2),
      // the A operand of PV(gt-2); products with different accumulators are not ordered against each other's
      // operand reads, so the latest PV issued (gt-2 inside an item, gt-1 at its start) must have completed.
      auto issue_s = [&](uint32_t gt, uint32_t pv_issued) -> bool {
        const int s = gt & 1;
        const uint32_t ph = (gt >> 1) & 1;
        if (pv_issued > 0 && !mbar_wait(&bars[PV_DONE0 + ((pv_issued - 1) & 1)], ((pv_issued - 1) >> 1) & 1)) return false;
        if (!mbar_wait(&bars[K_FULL0 + s], ph)) return false;
        tc_fence_after();
        const uint32_t kb = sb + K_OFF + s * kStageBytes;
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16_ss(tmem + s * kTile, umma_desc_k_sw128(sb + Q_OFF + h * 16384 + k * 32),
                         umma_desc_k_sw128(kb + h * kHalfBytes + k * 32), idesc_s, (h | k) ? 1u : 0u);
        umma_commit(&bars[K_EMPTY0 + s]);
        umma_commit(&bars[S_FULL0 + s]);
        return true;
      };
      bool ok = true;
      for (long long w = blockIdx.x; w < total && ok; w += gridDim.x) {
        const Item it = read_item(p, w);
        if (!it.valid) continue;
        if (!mbar_wait(&bars[Q_FULL], n_item & 1) || *abort_flag) { fail(NF_ST_TIMEOUT_SMEM_FULL); break; }
        if (!issue_s(g, g)) { fail(NF_ST_TIMEOUT_SMEM_FULL); break; }
        for (int t = 0; t < it.n_tiles; ++t) {
          const uint32_t gt = g + t;
          if (t + 1 < it.n_tiles) {
            if (!issue_s(gt + 1, gt)) { fail(NF_ST_TIMEOUT_SMEM_FULL); ok = false; break; }
          } else {
            umma_commit(&bars[Q_EMPTY]);     // the last S product of the item has been issued
          }
          // the previous item's O must have been read out before this item's first PV overwrites it
          if (t == 0 && !mbar_wait(&bars[O_FREE], (n_item & 1) ^ 1)) { fail(NF_ST_TIMEOUT_TMEM_EMPTY); ok = false; break; }
          const int s = gt & 1;
          if (!mbar_wait(&bars[P_FULL0 + s], (gt >> 1) & 1) || !mbar_wait(&bars[V_FULL0 + s], (gt >> 1) & 1) || *abort_flag) {
            fail(NF_ST_TIMEOUT_SMEM_FULL);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t vb = sb + V_OFF + s * kStageBytes;
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16_ts(tmem + 2 * kTile, tmem + s * kTile + k * 8,      // P(t): 16 tokens = 8 columns per step
                         umma_desc_mn_sw128(vb + k * 2048, kHalfBytes, 1024), idesc_o, (t | k) ? 1u : 0u);
          umma_commit(&bars[V_EMPTY0 + s]);
          umma_commit(&bars[PV_DONE0 + s]);
        }
        g += it.n_tiles;
        ++n_item;
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax (one thread per query row)
    const int row = warp * 32 + lane;                  // query row = TMEM lane
    const uint32_t t_lane = tmem + (static_cast<uint32_t>(warp * 32) << 16);
    __nv_bfloat16* outp = reinterpret_cast<__nv_bfloat16*>(p.out);
    const float scale = p.sm_scale * kLog2e;
    uint32_t g = 0, n_item = 0;
    bool ok = true;
    for (long long w = blockIdx.x; w < total && ok; w += gridDim.x) {
      const Item it = read_item(p, w);
      if (!it.valid) continue;
      const int tl = row / group, hh = row % group;
      const bool row_valid = tl < it.ntok;
      const int pos = row_valid ? it.kv_len - (it.q_end - (it.tok0 + tl)) : -1;
      float m_ref = -INFINITY, l = 0.f;
      for (int t = 0; t < it.n_tiles; ++t) {
        const uint32_t gt = g + t;
        const int s = gt & 1;
        if (!mbar_wait(&bars[S_FULL0 + s], (gt >> 1) & 1) || *abort_flag) { fail(NF_ST_TIMEOUT_TMEM_FULL); ok = false; break; }
        tc_fence_after();
        uint32_t r0[32], r1[32];
        tmem_ld_32x32b_x32(t_lane + s * kTile, r0);
        tmem_ld_32x32b_x32(t_lane + s * kTile + 32, r1);
        tmem_ld_wait();
        const int cbase = t * kTile;
        if (cbase + kTile - 1 > pos) {                        // only tiles on the diagonal need the mask
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (cbase + j > pos) r0[j] = 0xff800000u;         // -inf
            if (cbase + 32 + j > pos) r1[j] = 0xff800000u;
          }
        }
        float mxp = -INFINITY;
#pragma unroll
        for (int j = 0; j < 32; ++j) mxp = fmaxf(mxp, fmaxf(__uint_as_float(r0[j]), __uint_as_float(r1[j])));
        const float mx = mxp * scale;
        const bool grow = mx > m_ref + kRescaleGap || (m_ref == -INFINITY && mx > -INFINITY);
        if (t == 0) {
          m_ref = mx;
        } else if (__any_sync(0xffffffffu, grow)) {
          // bring O (in TMEM) and the row sum to the new reference maximum; warp-wide because the TMEM
          // accesses are, rows that did not grow scale by one. O may only be touched between two PV
          // products: PV(t-1) is the last one issued (PV(t) needs this tile's P), so once it is done O is still
          if (!mbar_wait(&bars[PV_DONE0 + ((gt - 1) & 1)], ((gt - 1) >> 1) & 1) || *abort_flag) {
            fail(NF_ST_TIMEOUT_TMEM_FULL);
            ok = false;
            break;
          }
          tc_fence_after();
          const float alpha = grow ? (m_ref == -INFINITY ? 0.f : fast_exp2(m_ref - mx)) : 1.f;
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t ov[32];
            tmem_ld_32x32b_x32(t_lane + 2 * kTile + c * 32, ov);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) ov[j] = __float_as_uint(__uint_as_float(ov[j]) * alpha);
            tmem_st_32x32b_x32(t_lane + 2 * kTile + c * 32, ov);
          }
          tmem_st_wait();
          l *= alpha;
          if (grow) m_ref = mx;
        }
        const float ms = m_ref == -INFINITY ? 0.f : m_ref;
        float rs = 0.f;
        uint32_t pk[32];                                      // column j: tokens 2j, 2j + 1 of the tile
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float x0 = fast_exp2(fmaf(__uint_as_float(r0[2 * j]), scale, -ms));
          const float x1 = fast_exp2(fmaf(__uint_as_float(r0[2 * j + 1]), scale, -ms));
          const float y0 = fast_exp2(fmaf(__uint_as_float(r1[2 * j]), scale, -ms));
          const float y1 = fast_exp2(fmaf(__uint_as_float(r1[2 * j + 1]), scale, -ms));
          rs += (x0 + x1) + (y0 + y1);
          pk[j] = pack_bf16x2(x0, x1);
          pk[16 + j] = pack_bf16x2(y0, y1);
        }
        l += rs;
        // P(t) goes over the first half of the S accumulator it was computed from (all 64 scores are in
        // registers); the other accumulator holds P(t-1) / S(t+1), so nothing has to be waited for
        tmem_st_32x32b_x32(t_lane + s * kTile, pk);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[P_FULL0 + s]);
      }
      if (!ok) break;
      g += it.n_tiles;
      // ---- the item's last PV product, then O / l to global memory ----
      // (one barrier per S accumulator: the softmax warps do not wait for every product, and up to two can be
      // outstanding here, which a single barrier's phase bit could not tell apart)
      if (!mbar_wait(&bars[PV_DONE0 + ((g - 1) & 1)], ((g - 1) >> 1) & 1) || *abort_flag) { fail(NF_ST_TIMEOUT_TMEM_FULL); break; }
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = outp + (static_cast<long long>(it.tok0 + tl) * p.q_heads + it.kvh * group + hh) * HD;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_lane + 2 * kTile + c * 32, r);
        tmem_ld_wait();
        if (row_valid) {
#pragma unroll
          for (int g8 = 0; g8 < 4; ++g8) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(r[g8 * 8 + 0]) * inv, __uint_as_float(r[g8 * 8 + 1]) * inv);
            v.y = pack_bf16x2(__uint_as_float(r[g8 * 8 + 2]) * inv, __uint_as_float(r[g8 * 8 + 3]) * inv);
            v.z = pack_bf16x2(__uint_as_float(r[g8 * 8 + 4]) * inv, __uint_as_float(r[g8 * 8 + 5]) * inv);
            v.w = pack_bf16x2(__uint_as_float(r[g8 * 8 + 6]) * inv, __uint_as_float(r[g8 * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + c * 32 + g8 * 8) = v;
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[O_FREE]);
      ++n_item;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem, 256);
  }
}

}  // namespace
}  // namespace nf

extern "C" int nfk_attn_prefill_ws(const nfk_attn_params* p, cudaStream_t stream) {
  using namespace nf;
  if (p == nullptr) return NF_ERR_BAD_ARG;
  if (!p->q || !p->out || !p->kv_pool || !p->qo_indptr || !p->kv_indptr || !p->kv_indices || !p->kv_last_page_len)
    return NF_ERR_BAD_ARG;
  if (p->kv_heads <= 0 || p->q_heads % p->kv_heads != 0 || p->num_pages <= 0) return NF_ERR_BAD_ARG;
  const int group = p->q_heads / p->kv_heads;
  if (p->head_dim != HD || p->page_size != kPage || group > 16 || (16 % group) != 0) return NF_ERR_UNSUPPORTED;
  if (p->num_items == 0) return NF_OK;
  if (p->num_items < 0 || p->items == nullptr) return NF_ERR_BAD_ARG;
  // Q as [tokens * q_heads][128] (the token count is not known here: any row the items name is inside
  // the caller's buffer, the map's row bound only has to be large enough); the pool as
  // [pages * 2 * kv_heads * 16][128]. Boxes: the `group` rows of one token, one page of one head; 64 columns.
  CUtensorMap tmQ, tmKV;
  int rc = make_tmap_bf16_2d(&tmQ, p->q, 1ull << 26, HD, HD, static_cast<uint32_t>(group), 64);
  if (rc != NF_OK) return rc;
  rc = make_tmap_bf16_2d(&tmKV, p->kv_pool, static_cast<uint64_t>(p->num_pages) * 2 * p->kv_heads * kPage, HD, HD, kPage, 64);
  if (rc != NF_OK) return rc;
  static bool attr_dev[kMaxDevices] = {false};   // the attribute is per device
  bool& attr = attr_dev[device_slot()];
  if (!attr) {
    if (cudaFuncSetAttribute(attn_prefill_ws_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) !=
        cudaSuccess)
      return NF_ERR_CUDA;
    attr = true;
  }
  const long long total = static_cast<long long>(p->num_items) * p->kv_heads;
  long long ctas = p->num_ctas > 0 ? p->num_ctas : 2LL * device_sm_count();   // two resident CTAs per SM
  if (ctas > total) ctas = total;
  attn_prefill_ws_kernel<<<static_cast<int>(ctas), kThreads, kSmemBytes, stream>>>(tmQ, tmKV, *p);
  return cudaGetLastError() == cudaSuccess ? NF_OK : NF_ERR_CUDA;
}
