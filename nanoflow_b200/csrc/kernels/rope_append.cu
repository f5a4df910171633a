// Fused split + rotary embedding + paged-KV append, one pass over the packed QKV activations:
//   q_out[t, h, :]            = rope(q[t, h, :], pos[t])
//   pool[page(t), K, h, slot] = rope(k[t, h, :], pos[t])
//   pool[page(t), V, h, slot] = v[t, h, :]
// page(t) = kv_indices[kv_indptr[req(t)] + pos[t] / page_size], slot = pos[t] % page_size.
// Rotation pairs element i with i + head_dim/2 (the Hugging Face Llama convention); the inverse
// frequencies come from the host so Llama-3.1 style frequency scaling needs no device code.
// A (token, head) unit is handled by head_dim/16 threads, each moving two 16-byte vectors. Two forms:
// a CTA handles one token at a time and builds that token's cos / sin table in shared memory, or
// (when the caller supplies the iteration's table from nfk_rope_table) the units are spread flat over
// the grid and the angles are read.
//
// Counterpart in the reference: splitRopeAppendKernel, pipeline/include/small_cuda_operator.cuh:21-93.
#include "common.cuh"
#include "kernels.h"

namespace nf {
namespace {

// One CTA per token (grid-stride). The token's cos / sin table (head_dim/2 entries) is computed once
// into shared memory with full-range sincosf and then shared by all heads, so the expensive
// argument reduction runs head_dim/2 times per token instead of once per (head, element).
__global__ void __launch_bounds__(256)
rope_append_kernel(nfk_rope_append_params p) {
  __shared__ float s_cos[128], s_sin[128];
  const int hd = p.head_dim;
  const int half = hd >> 1;
  const int lph = hd >> 4;  // threads per (token, head) unit
  const int heads_total = p.q_heads + 2 * p.kv_heads;
  const int units = heads_total * lph;
  const __nv_bfloat16* qkv = reinterpret_cast<const __nv_bfloat16*>(p.qkv);
  __nv_bfloat16* q_out = reinterpret_cast<__nv_bfloat16*>(p.q_out);
  __nv_bfloat16* pool = reinterpret_cast<__nv_bfloat16*>(p.kv_pool);

  for (int t = blockIdx.x; t < p.T; t += gridDim.x) {
    const int pos = p.positions[t];
    __syncthreads();   // previous token's table is no longer in use
    for (int i = threadIdx.x; i < half; i += blockDim.x)
      sincosf(static_cast<float>(pos) * p.inv_freq[i], &s_sin[i], &s_cos[i]);
    __syncthreads();
    const __nv_bfloat16* row = qkv + static_cast<long long>(t) * p.ld_qkv;
    // page slot of this token (shared by all kv heads)
    const int b = p.token_req[t];
    const int pg_slot = p.kv_indptr[b] + pos / p.page_size;
    const int page = (pos >= 0 && pg_slot < p.kv_indptr[b + 1]) ? p.kv_indices[pg_slot] : -1;
    const bool page_ok = page >= 0 && page < p.num_pages;
    if (!page_ok && threadIdx.x == 0) report_status(p.status, NF_ST_BAD_INDEX);
    const int slot = pos % p.page_size;

    for (int u = threadIdx.x; u < units; u += blockDim.x) {
      const int h = u / lph;
      const int l = u % lph;
      int kind, hh;  // 0 = q, 1 = k, 2 = v
      const __nv_bfloat16* src;
      if (h < p.q_heads) {
        kind = 0; hh = h; src = row + p.q_off + hh * hd;
      } else if (h < p.q_heads + p.kv_heads) {
        kind = 1; hh = h - p.q_heads; src = row + p.k_off + hh * hd;
      } else {
        kind = 2; hh = h - p.q_heads - p.kv_heads; src = row + p.v_off + hh * hd;
      }
      __nv_bfloat16* dst;
      if (kind == 0) {
        dst = q_out + (static_cast<long long>(t) * p.q_heads + hh) * hd;
      } else {
        if (!page_ok) continue;  // skip the write; never touch memory outside the pool
        dst = pool + ((((static_cast<long long>(page) * 2 + (kind - 1)) * p.kv_heads + hh) *
                       p.page_size + slot) * hd);
      }
      const uint4 lo = *reinterpret_cast<const uint4*>(src + 8 * l);
      const uint4 hi = *reinterpret_cast<const uint4*>(src + half + 8 * l);
      if (kind == 2) {
        *reinterpret_cast<uint4*>(dst + 8 * l) = lo;
        *reinterpret_cast<uint4*>(dst + half + 8 * l) = hi;
        continue;
      }
      const uint32_t lw[4] = {lo.x, lo.y, lo.z, lo.w}, hw[4] = {hi.x, hi.y, hi.z, hi.w};
      uint32_t ol[4], oh[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 a = unpack_bf16x2(lw[j]), bb = unpack_bf16x2(hw[j]);
        const float c0 = s_cos[8 * l + 2 * j], s0 = s_sin[8 * l + 2 * j];
        const float c1 = s_cos[8 * l + 2 * j + 1], s1 = s_sin[8 * l + 2 * j + 1];
        ol[j] = pack_bf16x2(a.x * c0 - bb.x * s0, a.y * c1 - bb.y * s1);
        oh[j] = pack_bf16x2(bb.x * c0 + a.x * s0, bb.y * c1 + a.y * s1);
      }
      *reinterpret_cast<uint4*>(dst + 8 * l) = make_uint4(ol[0], ol[1], ol[2], ol[3]);
      *reinterpret_cast<uint4*>(dst + half + 8 * l) = make_uint4(oh[0], oh[1], oh[2], oh[3]);
    }
  }
}

// Same work with the angles read from a per-iteration table: no per-token set-up, so the
// (token, head, 16-byte pair) units are spread flat over the grid and the kernel is a pure copy.
__global__ void __launch_bounds__(256)
rope_append_table_kernel(nfk_rope_append_params p) {
  const int hd = p.head_dim;
  const int half = hd >> 1;
  const int lph = hd >> 4;
  const int heads_total = p.q_heads + 2 * p.kv_heads;
  const int units = heads_total * lph;
  const __nv_bfloat16* qkv = reinterpret_cast<const __nv_bfloat16*>(p.qkv);
  __nv_bfloat16* q_out = reinterpret_cast<__nv_bfloat16*>(p.q_out);
  __nv_bfloat16* pool = reinterpret_cast<__nv_bfloat16*>(p.kv_pool);
  const long long total = static_cast<long long>(p.T) * units;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < total; i += 256ll * gridDim.x) {
    const int t = static_cast<int>(i / units);
    const int u = static_cast<int>(i - static_cast<long long>(t) * units);
    const int h = u / lph, l = u % lph;
    const __nv_bfloat16* row = qkv + static_cast<long long>(t) * p.ld_qkv;
    int kind, hh;
    const __nv_bfloat16* src;
    if (h < p.q_heads) {
      kind = 0; hh = h; src = row + p.q_off + hh * hd;
    } else if (h < p.q_heads + p.kv_heads) {
      kind = 1; hh = h - p.q_heads; src = row + p.k_off + hh * hd;
    } else {
      kind = 2; hh = h - p.q_heads - p.kv_heads; src = row + p.v_off + hh * hd;
    }
    __nv_bfloat16* dst;
    if (kind == 0) {
      dst = q_out + (static_cast<long long>(t) * p.q_heads + hh) * hd;
    } else {
      const int pos = p.positions[t];
      const int b = p.token_req[t];
      const int pg_slot = p.kv_indptr[b] + pos / p.page_size;
      const int page = (pos >= 0 && pg_slot < p.kv_indptr[b + 1]) ? p.kv_indices[pg_slot] : -1;
      if (page < 0 || page >= p.num_pages) {   // never touch memory outside the pool
        if (l == 0 && hh == 0) report_status(p.status, NF_ST_BAD_INDEX);
        continue;
      }
      dst = pool + ((((static_cast<long long>(page) * 2 + (kind - 1)) * p.kv_heads + hh) * p.page_size +
                     pos % p.page_size) * hd);
    }
    const uint4 lo = *reinterpret_cast<const uint4*>(src + 8 * l);
    const uint4 hi = *reinterpret_cast<const uint4*>(src + half + 8 * l);
    if (kind == 2) {
      *reinterpret_cast<uint4*>(dst + 8 * l) = lo;
      *reinterpret_cast<uint4*>(dst + half + 8 * l) = hi;
      continue;
    }
    const float4* cs = reinterpret_cast<const float4*>(p.cos_sin + (static_cast<long long>(t) * half + 8 * l) * 2);
    const uint32_t lw[4] = {lo.x, lo.y, lo.z, lo.w}, hw[4] = {hi.x, hi.y, hi.z, hi.w};
    uint32_t ol[4], oh[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float4 c = cs[j];   // (cos, sin) of elements 8l+2j and 8l+2j+1
      const float2 a = unpack_bf16x2(lw[j]), bb = unpack_bf16x2(hw[j]);
      ol[j] = pack_bf16x2(a.x * c.x - bb.x * c.y, a.y * c.z - bb.y * c.w);
      oh[j] = pack_bf16x2(bb.x * c.x + a.x * c.y, bb.y * c.z + a.y * c.w);
    }
    *reinterpret_cast<uint4*>(dst + 8 * l) = make_uint4(ol[0], ol[1], ol[2], ol[3]);
    *reinterpret_cast<uint4*>(dst + half + 8 * l) = make_uint4(oh[0], oh[1], oh[2], oh[3]);
  }
}

__global__ void __launch_bounds__(256)
rope_table_kernel(nfk_rope_table_params p) {
  const long long total = static_cast<long long>(p.T) * p.half;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < total; i += 256ll * gridDim.x) {
    const int t = static_cast<int>(i / p.half);
    const int k = static_cast<int>(i - static_cast<long long>(t) * p.half);
    float s, c;
    sincosf(static_cast<float>(p.positions[t]) * p.inv_freq[k], &s, &c);
    reinterpret_cast<float2*>(p.cos_sin)[i] = make_float2(c, s);
  }
}

}  // namespace
}  // namespace nf

extern "C" int nfk_rope_table(const nfk_rope_table_params* p, cudaStream_t stream) {
  using namespace nf;
  if (p == nullptr) return NF_ERR_BAD_ARG;
  if (p->T == 0) return NF_OK;
  if (!p->cos_sin || !p->inv_freq || !p->positions || p->T < 0 || p->half <= 0 || p->half % 8 != 0 ||
      (reinterpret_cast<uintptr_t>(p->cos_sin) & 15))
    return NF_ERR_BAD_ARG;
  const long long total = static_cast<long long>(p->T) * p->half;
  long long blocks = (total + 255) / 256;
  if (blocks > device_sm_count() * 8) blocks = device_sm_count() * 8;
  rope_table_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(*p);
  return cudaGetLastError() == cudaSuccess ? NF_OK : NF_ERR_CUDA;
}

extern "C" int nfk_rope_append(const nfk_rope_append_params* p, cudaStream_t stream) {
  using namespace nf;
  if (p == nullptr) return NF_ERR_BAD_ARG;
  if (p->T == 0) return NF_OK;
  if (!p->qkv || !p->q_out || !p->kv_pool || !p->inv_freq || !p->positions || !p->token_req ||
      !p->kv_indptr || !p->kv_indices)
    return NF_ERR_BAD_ARG;
  if (p->T < 0 || p->head_dim % 16 != 0 || p->head_dim > 256 || p->page_size <= 0 ||
      p->ld_qkv % 8 != 0 || p->q_off % 8 != 0 || p->k_off % 8 != 0 || p->v_off % 8 != 0 ||
      (reinterpret_cast<uintptr_t>(p->qkv) & 15) || (reinterpret_cast<uintptr_t>(p->q_out) & 15) ||
      (reinterpret_cast<uintptr_t>(p->kv_pool) & 15))
    return NF_ERR_BAD_ARG;
  const int units = (p->q_heads + 2 * p->kv_heads) * (p->head_dim / 16);
  if (p->cos_sin != nullptr) {
    if (reinterpret_cast<uintptr_t>(p->cos_sin) & 15) return NF_ERR_BAD_ARG;
    const long long total = static_cast<long long>(p->T) * units;
    long long nb = (total + 255) / 256;
    if (nb > device_sm_count() * 16) nb = device_sm_count() * 16;
    rope_append_table_kernel<<<static_cast<int>(nb), 256, 0, stream>>>(*p);
    return cudaGetLastError() == cudaSuccess ? NF_OK : NF_ERR_CUDA;
  }
  int threads = units < 64 ? 64 : (units < 128 ? 128 : 256);
  int blocks = p->T < device_sm_count() * 8 ? p->T : device_sm_count() * 8;
  rope_append_kernel<<<blocks, threads, 0, stream>>>(*p);
  return cudaGetLastError() == cudaSuccess ? NF_OK : NF_ERR_CUDA;
}
