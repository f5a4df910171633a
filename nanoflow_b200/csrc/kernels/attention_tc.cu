// Chunked-prefill attention on the 5th-generation tensor cores (head_dim 128).
//
// A work item is (request, first token, token count <= 128/group) x kv head, as in nfk_attn_prefill:
// the item's query rows r = token * group + head fill one 128-row MMA tile. Per 64-token KV tile:
//
//   S[128 x 64]  = Q K^T          tcgen05.mma, Q and K staged K-major / 128B-swizzled in shared memory,
//                                 accumulator in TMEM columns [0, 64)
//   P            = exp2(S*scale - m)   two threads per row read the halves of its S row from TMEM, keep the
//                                 running max / sum, write P (bf16) back to shared memory as the next A operand
//   O[128 x 128] += P V           tcgen05.mma accumulating in TMEM columns [64, 192) across the tiles; V
//                                 arrives token-major, so the tile is first transposed shared->shared
//                                 (ldmatrix.trans + stmatrix) into the K-major form the B operand needs
//
// The accumulator stays in TMEM for the whole item: P is taken relative to a reference maximum that
// is only moved (and O rescaled in TMEM, tcgen05.ld / tcgen05.st) when a row's maximum outgrows it
// by more than 2^8, which after the first tiles is rare; the row sum is kept in fp32 and divides the
// result at the end. K / V pages are gathered with cp.async (16-byte chunks placed directly in the
// swizzled layouts); the next tile's loads are issued as soon as this tile's K and V have been
// consumed (after the S product and the transposes) and run under its softmax and PV product. Two
// 256-thread CTAs share an SM (97 KB of shared memory and 256 TMEM columns each), so one CTA's
// softmax runs under the other's MMAs. Every wait on an
// mbarrier is bounded and failures end in the status word.
//
// Takes the place of the reference's FlashInfer BatchPrefillWithPagedKVCacheKernel
// (gemv/include/attention/prefill.cuh:1066-1374, mma.sync m16n16k16 + ldmatrix on sm_80).
#include "common.cuh"
#include "kernels.h"

namespace nf {
namespace {

constexpr int HD = 128;
constexpr int kPage = 16;
constexpr int kTile = 64;            // kv tokens per tile
constexpr int kThreads = 256;        // two per query row: warps 0-3 take the first half of a row's columns,
                                     // warps 4-7 the second (a warp reaches the 32 TMEM lanes of its index mod 4)
constexpr float kLog2e = 1.4426950408889634f;

// shared-memory map (bytes from a 1024-aligned base); every MMA operand region is 1024-aligned
constexpr int Q_OFF = 0;                         // 2 halves x [128 rows][64 hd]   32 KB
constexpr int K_OFF = 32768;                     // 2 halves x [64 tok][64 hd]     16 KB
constexpr int V_OFF = K_OFF + 16384;             // [64 tok][128 hd] (token-major) 16 KB
constexpr int VT_OFF = V_OFF + 16384;            // [128 hd][64 tok]               16 KB
constexpr int P_OFF = VT_OFF + 16384;            // [128 rows][64 tok]             16 KB
constexpr int BAR_OFF = P_OFF + 16384;
constexpr int EXCH_OFF = BAR_OFF + 64;           // [2 halves][128 rows] fp32: what the two threads of a row exchange
constexpr int kSmemBytes = EXCH_OFF + 1024 + 1024;  // + alignment slack
constexpr float kRescaleGap = 8.0f;              // log2 of how far a row maximum may outgrow its reference

__device__ __forceinline__ void cp_async16(uint32_t smem_addr, const void* gptr) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr), "l"(gptr) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// K-major, 128B-swizzled operand tile: rows of 64 bf16 (128 bytes); the 16-byte chunk c of row r
// sits at chunk position c ^ (r % 8) (what TMA SWIZZLE_128B would produce and the UMMA descriptor of
// umma_desc_k_sw128 expects).
__device__ __forceinline__ uint32_t sw128(int row, int chunk) {
  return static_cast<uint32_t>(row * 128 + ((chunk ^ (row & 7)) << 4));
}

__global__ void __launch_bounds__(kThreads, 2)
attn_prefill_tc_kernel(nfk_attn_params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const uint32_t sb = smem_u32(smem);
  uint64_t* bar_s = reinterpret_cast<uint64_t*>(smem + BAR_OFF);
  uint64_t* bar_o = bar_s + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_s + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile float* exch = reinterpret_cast<volatile float*>(smem + EXCH_OFF);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int half = warp >> 2;                       // which half of the row's columns this thread handles
  const int row = (warp & 3) * 32 + lane;           // query row = TMEM lane

  if (threadIdx.x == 0) {
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, 256);   // S: columns [0,64), O: columns [64,192)
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t t_lane = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
  const uint32_t t_s = t_lane + half * 32;          // this thread's 32 S columns
  const uint32_t t_o = t_lane + 64 + half * 64;     // this thread's 64 O columns
  const uint32_t idesc_s = umma_idesc_bf16(128, kTile), idesc_o = umma_idesc_bf16(128, HD);
  uint32_t ph_s = 0, ph_o = 0;

  const int group = p.q_heads / p.kv_heads;
  const long long total = static_cast<long long>(p.num_items) * p.kv_heads;
  const __nv_bfloat16* qbase = reinterpret_cast<const __nv_bfloat16*>(p.q);
  const __nv_bfloat16* pool = reinterpret_cast<const __nv_bfloat16*>(p.kv_pool);
  __nv_bfloat16* outp = reinterpret_cast<__nv_bfloat16*>(p.out);
  const float scale = p.sm_scale * kLog2e;
  bool alive = true;

  for (long long w = blockIdx.x; w < total && alive; w += gridDim.x) {
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
    const int kv_hi = kv_len - (q_end - (tok0 + ntok - 1)) + 1;   // keys visible to the last row
    if (ntok <= 0 || np <= 0 || kv_hi <= 0) continue;             // uniform across the CTA
    const int n_tiles = (kv_hi + kTile - 1) / kTile;

    const int tl = row / group, hh = row % group;                  // this thread's query row
    const bool row_valid = tl < ntok;
    const int pos = row_valid ? kv_len - (q_end - (tok0 + tl)) : -1;

    // ---- Q tile: 128 rows x 16 chunks, zero rows past the item ----
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int idx = threadIdx.x + kThreads * j;
      const int r = idx >> 4, c = idx & 15;
      const int rt = r / group;
      const uint32_t dst = sb + Q_OFF + (c >> 3) * 16384 + sw128(r, c & 7);
      if (rt < ntok) {
        cp_async16(dst, qbase + (static_cast<long long>(tok0 + rt) * p.q_heads + kvh * group + r % group) * HD + c * 8);
      } else {
        st_shared_v4(dst, 0u, 0u, 0u, 0u);
      }
    }
    // ---- K / V tile loader: 64 tokens x 16 chunks each ----
    auto issue = [&](int t) {
      if (t < n_tiles) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int idx = threadIdx.x + kThreads * j;
          const int r = idx >> 4, c = idx & 15;
          int pslot = t * (kTile / kPage) + r / kPage;
          if (pslot >= np) pslot = 0;   // past the sequence: a valid page, masked below
          int page = p.kv_indices[pg0 + pslot];
          if (page < 0 || page >= p.num_pages) {
            report_status(p.status, NF_ST_BAD_INDEX);
            page = 0;
          }
          const __nv_bfloat16* kp = pool + ((static_cast<long long>(page) * 2) * p.kv_heads + kvh) * (kPage * HD) +
                                    (r % kPage) * HD + c * 8;
          cp_async16(sb + K_OFF + (c >> 3) * 8192 + sw128(r, c & 7), kp);
          cp_async16(sb + V_OFF + r * 256 + ((c ^ (r & 7)) << 4), kp + static_cast<long long>(p.kv_heads) * (kPage * HD));
        }
      }
      cp_async_commit();
    };
    issue(0);

    float m_ref = -INFINITY, l = 0.f;   // l: this thread's half of the row sum

    for (int t = 0; t < n_tiles; ++t) {
      cp_async_wait<0>();
      fence_proxy_async_smem();
      __syncthreads();
      // ---- S = Q K^T ----
      if (threadIdx.x == 0) {
        tc_fence_after();
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16_ss(tmem, umma_desc_k_sw128(sb + Q_OFF + h * 16384 + k * 32),
                         umma_desc_k_sw128(sb + K_OFF + h * 8192 + k * 32), idesc_s, (h | k) ? 1u : 0u);
        umma_commit(bar_s);
      }
      __syncwarp();
      // The previous tile's PV product still reads V^T and P (and writes O) until bar_o fires.
      if (t > 0) {
        if (!mbar_wait(bar_o, ph_o)) {
          report_status(p.status, NF_ST_TIMEOUT_TMEM_FULL);
          *abort_flag = 1;
        }
        ph_o ^= 1;
        tc_fence_after();
      }
      // ---- V^T for the PV product: 8x8 blocks, ldmatrix.trans -> stmatrix (under the S MMAs);
      //      a warp takes four hd blocks (one per 8 lanes) x four token blocks ----
      {
        const uint32_t vsrc = sb + V_OFF;
        const int j = lane >> 3, i = lane & 7;
        const int hb = 4 * (warp & 3) + j;              // hd block of this lane's matrix
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int tb = 4 * half + q;
          uint32_t d0, d1, d2, d3;
          asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                       : "=r"(d0), "=r"(d1), "=r"(d2), "=r"(d3)
                       : "r"(vsrc + (tb * 8 + i) * 256 + ((hb ^ i) << 4)));
          const int hd = hb * 8 + i;
          asm volatile("stmatrix.sync.aligned.m8n8.x4.shared.b16 [%0], {%1,%2,%3,%4};" ::"r"(
                           sb + VT_OFF + sw128(hd, tb)),
                       "r"(d0), "r"(d1), "r"(d2), "r"(d3)
                       : "memory");
        }
      }
      if (!mbar_wait(bar_s, ph_s)) {
        report_status(p.status, NF_ST_TIMEOUT_TMEM_FULL);
        *abort_flag = 1;
      }
      ph_s ^= 1;
      tc_fence_after();
      // ---- softmax of this thread's half row ----
      uint32_t r0[32];
      tmem_ld_32x32b_x32(t_s, r0);
      tmem_ld_wait();
      const int cbase = t * kTile + half * 32;
      // Only the tile(s) on the diagonal need the causal mask; the row maximum is taken on the raw
      // scores (the scale is positive) and the scale folded into the exponent's multiply-add.
      if (cbase + 31 > pos) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (cbase + j > pos) r0[j] = 0xff800000u;        // -inf
      }
      float mxp = -INFINITY;
#pragma unroll
      for (int j = 0; j < 32; ++j) mxp = fmaxf(mxp, __uint_as_float(r0[j]));
      exch[half * 128 + row] = mxp;
      // K has been consumed by the S product and, once every warp is past its transposes, V too:
      // the next tile's loads start now and run under this tile's softmax and PV product.
      __syncthreads();
      issue(t + 1);
      {
        const float mx = fmaxf(mxp, exch[(half ^ 1) * 128 + row]) * scale;   // the same in both threads of the row
        // Reference maximum: follows the row maximum only when that outgrows it by 2^kRescaleGap;
        // then O (in TMEM) and the row sum are brought to the new reference. Warp-wide because the
        // TMEM accesses are; the two warps that share these rows take the same decision.
        const bool grow = mx > m_ref + kRescaleGap || (m_ref == -INFINITY && mx > -INFINITY);
        if (t == 0) {
          m_ref = mx;
        } else if (__any_sync(0xffffffffu, grow)) {
          const float alpha = grow ? (m_ref == -INFINITY ? 0.f : fast_exp2(m_ref - mx)) : 1.f;
#pragma unroll 1
          for (int c = 0; c < 2; ++c) {
            uint32_t ov[32];
            tmem_ld_32x32b_x32(t_o + c * 32, ov);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) ov[j] = __float_as_uint(__uint_as_float(ov[j]) * alpha);
            tmem_st_32x32b_x32(t_o + c * 32, ov);
          }
          tmem_st_wait();
          l *= alpha;
          if (grow) m_ref = mx;
        }
        const float ms = m_ref == -INFINITY ? 0.f : m_ref;
        float rs = 0.f;
        const uint32_t prow = sb + P_OFF;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t w0[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float x0 = fast_exp2(fmaf(__uint_as_float(r0[c * 8 + 2 * e]), scale, -ms));
            const float x1 = fast_exp2(fmaf(__uint_as_float(r0[c * 8 + 2 * e + 1]), scale, -ms));
            rs += x0 + x1;
            w0[e] = pack_bf16x2(x0, x1);
          }
          st_shared_v4(prow + sw128(row, half * 4 + c), w0[0], w0[1], w0[2], w0[3]);   // tokens 32*half + 8c ..
        }
        l += rs;
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncthreads();   // P and V^T are complete
      if (*abort_flag) {
        alive = false;
        break;
      }
      // ---- O += P V ----
      if (threadIdx.x == 0) {
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_bf16_ss(tmem + 64, umma_desc_k_sw128(sb + P_OFF + k * 32), umma_desc_k_sw128(sb + VT_OFF + k * 32),
                       idesc_o, (t | k) ? 1u : 0u);
        umma_commit(bar_o);
      }
      __syncwarp();
    }
    cp_async_wait<0>();
    if (alive) {
      if (!mbar_wait(bar_o, ph_o)) {
        report_status(p.status, NF_ST_TIMEOUT_TMEM_FULL);
        *abort_flag = 1;
      }
      ph_o ^= 1;
      tc_fence_after();
      exch[half * 128 + row] = l;
      __syncthreads();
      const float lsum = l + exch[(half ^ 1) * 128 + row];
      const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
      __nv_bfloat16* dst = outp + (static_cast<long long>(tok0 + tl) * p.q_heads + kvh * group + hh) * HD + half * 64;
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_o + c * 32, r);
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
    }
    __syncthreads();   // Q, S, O and the exchange words are rewritten by the next item
    if (*abort_flag) alive = false;
  }

  cp_async_wait<0>();
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 256);
  }
}

inline int sm_count_tc() { return device_sm_count(); }

}  // namespace
}  // namespace nf

extern "C" int nfk_attn_prefill_tc(const nfk_attn_params* p, cudaStream_t stream) {
  using namespace nf;
  if (p == nullptr) return NF_ERR_BAD_ARG;
  if (!p->q || !p->out || !p->kv_pool || !p->qo_indptr || !p->kv_indptr || !p->kv_indices || !p->kv_last_page_len)
    return NF_ERR_BAD_ARG;
  if (p->kv_heads <= 0 || p->q_heads % p->kv_heads != 0) return NF_ERR_BAD_ARG;
  const int group = p->q_heads / p->kv_heads;
  if (p->head_dim != HD || p->page_size != kPage || group > 16 || (16 % group) != 0) return NF_ERR_UNSUPPORTED;
  if (p->num_items == 0) return NF_OK;
  if (p->num_items < 0 || p->items == nullptr) return NF_ERR_BAD_ARG;
  static bool attr_dev[kMaxDevices] = {false};   // the attribute is per device
  bool& attr = attr_dev[device_slot()];
  if (!attr) {
    if (cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) !=
        cudaSuccess)
      return NF_ERR_CUDA;
    attr = true;
  }
  const long long total = static_cast<long long>(p->num_items) * p->kv_heads;
  long long ctas = p->num_ctas > 0 ? p->num_ctas : 2LL * sm_count_tc();   // two resident CTAs per SM
  if (ctas > total) ctas = total;
  attn_prefill_tc_kernel<<<static_cast<int>(ctas), kThreads, kSmemBytes, stream>>>(*p);
  return cudaGetLastError() == cudaSuccess ? NF_OK : NF_ERR_CUDA;
}
