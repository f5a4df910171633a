// Memory-bound helper kernels: RMSNorm (plain and residual-add fused), embedding gather with
// device-side token feedback, row gather, SiLU*mul, column-block copy, transpose, greedy arg-max
// sampling (single shard and cross-shard combine), a bounded sleep and device progress flags.
// All move data as 16-byte vectors and keep a row in registers so each byte crosses HBM once.
//
// Counterparts in the reference: pipeline/include/rms_norm.cuh:48-127 (rmsnorm_twoPassAlgo_e8),
// pipeline/src/small_cuda_operator.cu:9-24 (genEmbedding), :100-120 (silu_and_multiply_kernel),
// :133-152 (extractRankSubmatrixHalf), :165-205 (rowMaxKernel), :217-233 (copyLinesHalf),
// :64-83 (transposeKernel), pipeline/src/sleep.cu:5-11, pipeline/src/gemvDependency.cu:3-22.
#include "common.cuh"
#include "kernels.h"

namespace nf {
namespace {

constexpr int kNormThreads = 256;
constexpr int kNormMaxVec = 8;  // 8 vectors * 8 elements * 256 threads = 16384 columns

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  const int nw = blockDim.x >> 5;
  float t = (lane < nw) ? red[lane] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

template <bool ADD>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_kernel(__nv_bfloat16* __restrict__ out, __nv_bfloat16* resid,
               const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, int rows,
               int cols, float eps) {
  __shared__ float red[32];
  const int nvec = cols >> 3;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<long long>(row) * cols);
    uint4* rr = ADD ? reinterpret_cast<uint4*>(resid + static_cast<long long>(row) * cols) : nullptr;
    float v[kNormMaxVec][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
      const int vi = threadIdx.x + i * kNormThreads;
      if (vi < nvec) {
        const uint4 a = xr[vi];
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
        uint32_t bw[4] = {0, 0, 0, 0};
        if (ADD) {
          const uint4 b = rr[vi];
          bw[0] = b.x; bw[1] = b.y; bw[2] = b.z; bw[3] = b.w;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = unpack_bf16x2(aw[j]);
          if (ADD) {
            const float2 g = unpack_bf16x2(bw[j]);
            f.x += g.x;
            f.y += g.y;
          }
          v[i][2 * j] = f.x;
          v[i][2 * j + 1] = f.y;
        }
        if (ADD) {
          // The updated residual is stored in bf16; normalise what was stored so that the
          // residual stream and the normed activations stay consistent.
          uint4 o;
          o.x = pack_bf16x2(v[i][0], v[i][1]);
          o.y = pack_bf16x2(v[i][2], v[i][3]);
          o.z = pack_bf16x2(v[i][4], v[i][5]);
          o.w = pack_bf16x2(v[i][6], v[i][7]);
          rr[vi] = o;
          const uint32_t ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = unpack_bf16x2(ow[j]);
            v[i][2 * j] = f.x;
            v[i][2 * j + 1] = f.y;
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
      }
    }
    const float tot = block_sum(ss, red);
    const float inv = rsqrtf(tot / static_cast<float>(cols) + eps);
    uint4* orow = reinterpret_cast<uint4*>(out + static_cast<long long>(row) * cols);
    const uint4* wr = reinterpret_cast<const uint4*>(w);
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
      const int vi = threadIdx.x + i * kNormThreads;
      if (vi < nvec) {
        const uint4 ww = wr[vi];
        const uint32_t wv[4] = {ww.x, ww.y, ww.z, ww.w};
        uint32_t ov[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 g = unpack_bf16x2(wv[j]);
          ov[j] = pack_bf16x2(v[i][2 * j] * inv * g.x, v[i][2 * j + 1] * inv * g.y);
        }
        orow[vi] = make_uint4(ov[0], ov[1], ov[2], ov[3]);
      }
    }
  }
}

__global__ void embedding_kernel(__nv_bfloat16* __restrict__ out,
                                 const __nv_bfloat16* __restrict__ table,
                                 const int* __restrict__ host_ids,
                                 const int* __restrict__ feedback_src,
                                 const int* __restrict__ prev_tokens, int* ids_out, int n_tokens,
                                 int hidden, int vocab, unsigned int* status) {
  const int nvec = hidden >> 3;
  for (int t = blockIdx.x; t < n_tokens; t += gridDim.x) {
    int id = host_ids != nullptr ? host_ids[t] : 0;
    if (feedback_src != nullptr && prev_tokens != nullptr) {
      const int src = feedback_src[t];
      if (src >= 0) id = prev_tokens[src];
    }
    if (id < 0 || id >= vocab) {
      if (threadIdx.x == 0) report_status(status, NF_ST_BAD_INDEX);
      id = id < 0 ? 0 : vocab - 1;
    }
    if (threadIdx.x == 0 && ids_out != nullptr) ids_out[t] = id;
    const uint4* src = reinterpret_cast<const uint4*>(table + static_cast<long long>(id) * hidden);
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<long long>(t) * hidden);
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) dst[i] = src[i];
  }
}

__global__ void gather_rows_kernel(__nv_bfloat16* __restrict__ out,
                                   const __nv_bfloat16* __restrict__ in,
                                   const int* __restrict__ rows_idx, int n, int cols,
                                   long long ld_in, int in_rows, unsigned int* status) {
  const int nvec = cols >> 3;
  for (int r = blockIdx.x; r < n; r += gridDim.x) {
    int s = rows_idx[r];
    if (s < 0 || s >= in_rows) {
      if (threadIdx.x == 0) report_status(status, NF_ST_BAD_INDEX);
      s = s < 0 ? 0 : in_rows - 1;
    }
    const uint4* src = reinterpret_cast<const uint4*>(in + static_cast<long long>(s) * ld_in);
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<long long>(r) * cols);
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) dst[i] = src[i];
  }
}

__global__ void silu_mul_kernel(uint4* __restrict__ out, const uint4* __restrict__ gate,
                                const uint4* __restrict__ up, long long nvec) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint4 g = gate[i], u = up[i];
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 a = unpack_bf16x2(gw[j]), b = unpack_bf16x2(uw[j]);
      o[j] = pack_bf16x2(a.x / (1.f + __expf(-a.x)) * b.x, a.y / (1.f + __expf(-a.y)) * b.y);
    }
    out[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

__global__ void copy_cols_kernel(__nv_bfloat16* __restrict__ out, long long ld_out,
                                 const __nv_bfloat16* __restrict__ in, long long ld_in, int rows,
                                 int cols) {
  const int nvec = cols >> 3;
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const uint4* src = reinterpret_cast<const uint4*>(in + static_cast<long long>(r) * ld_in);
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<long long>(r) * ld_out);
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) dst[i] = src[i];
  }
}

__global__ void transpose_kernel(__nv_bfloat16* __restrict__ out,
                                 const __nv_bfloat16* __restrict__ in, int rows, int cols) {
  __shared__ __nv_bfloat16 tile[32][33];
  const int bx = blockIdx.x * 32, by = blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int r = by + j, c = bx + threadIdx.x;
    if (r < rows && c < cols) tile[j][threadIdx.x] = in[static_cast<long long>(r) * cols + c];
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int c = bx + j, r = by + threadIdx.x;
    if (r < rows && c < cols) out[static_cast<long long>(c) * rows + r] = tile[threadIdx.x][j];
  }
}

constexpr int kArgmaxThreads = 512;

__global__ void __launch_bounds__(kArgmaxThreads)
argmax_kernel(int* __restrict__ idx_out, float* __restrict__ val_out,
              const __nv_bfloat16* __restrict__ logits, int rows, int cols, long long ld,
              int col_offset) {
  __shared__ float s_val[kArgmaxThreads / 32];
  __shared__ int s_idx[kArgmaxThreads / 32];
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const __nv_bfloat16* lr = logits + static_cast<long long>(row) * ld;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    const int nvec = cols >> 3;
    const uint4* lv = reinterpret_cast<const uint4*>(lr);
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
      const uint4 a = lv[i];
      const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(aw[j]);
        const int c = i * 8 + 2 * j;
        if (f.x > best) { best = f.x; bi = c; }
        if (f.y > best) { best = f.y; bi = c + 1; }
      }
    }
    for (int c = (nvec << 3) + threadIdx.x; c < cols; c += blockDim.x) {
      const float f = __bfloat162float(lr[c]);
      if (f > best || (f == best && c < bi)) { best = f; bi = c; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { s_val[warp] = best; s_idx[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
      best = lane < kArgmaxThreads / 32 ? s_val[lane] : -INFINITY;
      bi = lane < kArgmaxThreads / 32 ? s_idx[lane] : 0x7fffffff;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
      }
      if (lane == 0) {
        if (bi == 0x7fffffff) bi = 0;  // all-NaN / -inf row
        idx_out[row] = bi + col_offset;
        if (val_out != nullptr) val_out[row] = best;
      }
    }
    __syncthreads();
  }
}

__global__ void argmax_combine_kernel(int* __restrict__ idx_out, const float* __restrict__ cand_val,
                                      const int* __restrict__ cand_idx, int shards, int rows) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  float best = cand_val[r];
  int bi = cand_idx[r];
  for (int s = 1; s < shards; ++s) {
    const float v = cand_val[static_cast<long long>(s) * rows + r];
    const int i = cand_idx[static_cast<long long>(s) * rows + r];
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
  }
  idx_out[r] = bi;
}

__global__ void sleep_kernel(long long nanos) {
  uint64_t t0, now;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
  for (int it = 0; it < (1 << 28); ++it) {
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
    if (static_cast<long long>(now - t0) >= nanos) break;
    __nanosleep(200);
  }
}

__global__ void flag_add_kernel(unsigned int* flag, unsigned int v) { atomicAdd(flag, v); }
__global__ void flag_clear_kernel(unsigned int* flag) { *flag = 0; }
__global__ void flag_wait_kernel(const unsigned int* flag, unsigned int target, long long nanos,
                                 unsigned int* status) {
  uint64_t t0, now;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
  for (int it = 0; it < (1 << 28); ++it) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v >= target) return;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
    if (static_cast<long long>(now - t0) >= nanos) break;
    __nanosleep(100);
  }
  report_status(status, NF_ST_TIMEOUT_PEER_FLAG);
}

inline int grid_for(int rows) {
  const int cap = device_sm_count() * 16;
  return rows < cap ? (rows > 0 ? rows : 1) : cap;
}
inline int ok_or_cuda() { return cudaGetLastError() == cudaSuccess ? NF_OK : NF_ERR_CUDA; }
inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace
}  // namespace nf

using namespace nf;
typedef __nv_bfloat16 bf16;

extern "C" int nfk_rmsnorm(void* out, const void* x, const void* w, int rows, int cols, float eps,
                           cudaStream_t stream) {
  if (rows == 0) return NF_OK;
  if (!out || !x || !w || rows < 0 || cols <= 0 || cols % 8 != 0 ||
      cols > kNormMaxVec * 8 * kNormThreads || !al16(out) || !al16(x) || !al16(w))
    return NF_ERR_BAD_ARG;
  rmsnorm_kernel<false><<<grid_for(rows), kNormThreads, 0, stream>>>(
      (bf16*)out, nullptr, (const bf16*)x, (const bf16*)w, rows, cols, eps);
  return ok_or_cuda();
}

extern "C" int nfk_add_rmsnorm(void* out, void* resid, const void* x, const void* w, int rows,
                               int cols, float eps, cudaStream_t stream) {
  if (rows == 0) return NF_OK;
  if (!out || !x || !w || !resid || rows < 0 || cols <= 0 || cols % 8 != 0 ||
      cols > kNormMaxVec * 8 * kNormThreads || !al16(out) || !al16(x) || !al16(w) || !al16(resid))
    return NF_ERR_BAD_ARG;
  rmsnorm_kernel<true><<<grid_for(rows), kNormThreads, 0, stream>>>(
      (bf16*)out, (bf16*)resid, (const bf16*)x, (const bf16*)w, rows, cols, eps);
  return ok_or_cuda();
}

extern "C" int nfk_embedding(void* out, const void* table, const int* host_ids,
                             const int* feedback_src, const int* prev_tokens, int* ids_out,
                             int n_tokens, int hidden, int vocab, unsigned int* status,
                             cudaStream_t stream) {
  if (n_tokens == 0) return NF_OK;
  if (!out || !table || n_tokens < 0 || hidden % 8 != 0 || vocab <= 0 || !al16(out) || !al16(table))
    return NF_ERR_BAD_ARG;
  if (host_ids == nullptr && (feedback_src == nullptr || prev_tokens == nullptr))
    return NF_ERR_BAD_ARG;
  embedding_kernel<<<grid_for(n_tokens), 128, 0, stream>>>((bf16*)out, (const bf16*)table, host_ids,
                                                           feedback_src, prev_tokens, ids_out,
                                                           n_tokens, hidden, vocab, status);
  return ok_or_cuda();
}

extern "C" int nfk_gather_rows(void* out, const void* in, const int* rows_idx, int n, int cols,
                               long long ld_in, unsigned int* status, int in_rows,
                               cudaStream_t stream) {
  if (n == 0) return NF_OK;
  if (!out || !in || !rows_idx || n < 0 || cols % 8 != 0 || ld_in % 8 != 0 || !al16(out) ||
      !al16(in) || in_rows <= 0)
    return NF_ERR_BAD_ARG;
  gather_rows_kernel<<<grid_for(n), 128, 0, stream>>>((bf16*)out, (const bf16*)in, rows_idx, n, cols,
                                                      ld_in, in_rows, status);
  return ok_or_cuda();
}

extern "C" int nfk_silu_mul(void* out, const void* gate, const void* up, long long n,
                            cudaStream_t stream) {
  if (n == 0) return NF_OK;
  if (!out || !gate || !up || n < 0 || n % 8 != 0 || !al16(out) || !al16(gate) || !al16(up))
    return NF_ERR_BAD_ARG;
  const long long nvec = n / 8;
  long long blocks = (nvec + 255) / 256;
  if (blocks > device_sm_count() * 8) blocks = device_sm_count() * 8;
  silu_mul_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>((uint4*)out, (const uint4*)gate,
                                                                (const uint4*)up, nvec);
  return ok_or_cuda();
}

extern "C" int nfk_copy_cols(void* out, long long ld_out, const void* in, long long ld_in, int rows,
                             int cols, cudaStream_t stream) {
  if (rows == 0 || cols == 0) return NF_OK;
  if (!out || !in || rows < 0 || cols % 8 != 0 || ld_out % 8 != 0 || ld_in % 8 != 0 || !al16(out) ||
      !al16(in))
    return NF_ERR_BAD_ARG;
  copy_cols_kernel<<<grid_for(rows), 128, 0, stream>>>((bf16*)out, ld_out, (const bf16*)in, ld_in,
                                                       rows, cols);
  return ok_or_cuda();
}

extern "C" int nfk_transpose(void* out, const void* in, int rows, int cols, cudaStream_t stream) {
  if (rows == 0 || cols == 0) return NF_OK;
  if (!out || !in || rows < 0 || cols < 0) return NF_ERR_BAD_ARG;
  dim3 grid((cols + 31) / 32, (rows + 31) / 32), block(32, 8);
  transpose_kernel<<<grid, block, 0, stream>>>((bf16*)out, (const bf16*)in, rows, cols);
  return ok_or_cuda();
}

extern "C" int nfk_argmax(int* idx_out, float* val_out, const void* logits, int rows, int cols,
                          long long ld, int col_offset, cudaStream_t stream) {
  if (rows == 0) return NF_OK;
  if (!idx_out || !logits || rows < 0 || cols <= 0 || ld % 8 != 0 || !al16(logits))
    return NF_ERR_BAD_ARG;
  argmax_kernel<<<grid_for(rows), kArgmaxThreads, 0, stream>>>(idx_out, val_out, (const bf16*)logits,
                                                               rows, cols, ld, col_offset);
  return ok_or_cuda();
}

extern "C" int nfk_argmax_combine(int* idx_out, const float* cand_val, const int* cand_idx,
                                  int shards, int rows, cudaStream_t stream) {
  if (rows == 0) return NF_OK;
  if (!idx_out || !cand_val || !cand_idx || shards <= 0 || rows < 0) return NF_ERR_BAD_ARG;
  argmax_combine_kernel<<<(rows + 127) / 128, 128, 0, stream>>>(idx_out, cand_val, cand_idx, shards,
                                                                rows);
  return ok_or_cuda();
}

extern "C" int nfk_sleep(int micros, cudaStream_t stream) {
  if (micros < 0 || micros > 1000000) return NF_ERR_BAD_ARG;
  sleep_kernel<<<1, 1, 0, stream>>>(static_cast<long long>(micros) * 1000);
  return ok_or_cuda();
}

extern "C" int nfk_flag_add(unsigned int* flag, unsigned int v, cudaStream_t stream) {
  if (!flag) return NF_ERR_BAD_ARG;
  flag_add_kernel<<<1, 1, 0, stream>>>(flag, v);
  return ok_or_cuda();
}
extern "C" int nfk_flag_clear(unsigned int* flag, cudaStream_t stream) {
  if (!flag) return NF_ERR_BAD_ARG;
  flag_clear_kernel<<<1, 1, 0, stream>>>(flag);
  return ok_or_cuda();
}
extern "C" int nfk_flag_wait(const unsigned int* flag, unsigned int target, int timeout_us,
                             unsigned int* status, cudaStream_t stream) {
  if (!flag || timeout_us <= 0 || timeout_us > 2000000) return NF_ERR_BAD_ARG;
  flag_wait_kernel<<<1, 1, 0, stream>>>(flag, target, static_cast<long long>(timeout_us) * 1000,
                                        status);
  return ok_or_cuda();
}
