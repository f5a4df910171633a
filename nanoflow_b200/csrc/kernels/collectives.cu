// Tensor-parallel collectives over a symmetric heap: every rank maps every peer's heap (CUDA IPC),
// so a buffer lives at the same byte offset on all GPUs and kernels reach peers with plain
// loads / stores over NVLink 5 through the NVSwitch (uniform bandwidth to every peer, hence direct
// one-step algorithms, no rings).
//
//   nfk_allreduce   sum of a bf16 [rows, cols] buffer over ranks. Row i is owned by rank i % nranks:
//                   the owner pulls the row from all ranks with 16-byte loads, adds in fp32 in rank
//                   order (deterministic), optionally adds its local residual row, and then any of:
//                   writes the sum to a local buffer (the residual stream stays sharded by owner),
//                   pushes the sum back into the buffer on every rank (classic in-place all-reduce),
//                   applies RMSNorm and pushes the normed row into a second symmetric buffer on every
//                   rank (reduce-scatter + norm + all-gather in one pass: the norm is computed once
//                   per row instead of once per rank and the pre-norm sum never crosses NVLink).
//   nfk_allgather   every rank pushes its shard of a symmetric buffer to all peers.
//   nfk_comm_barrier  cross-rank barrier.
//
// Synchronisation: per-op flag words in the symmetric heap, written by peers with st.release.sys
// and polled with ld.acquire.sys. Flags carry the caller's epoch (monotonic, e.g. the iteration
// number), so they are never reset. Every poll is bounded (~2 s); on expiry the kernel records
// NF_ST_TIMEOUT_PEER_FLAG in the status word, stops waiting and returns, so a dead peer shows up
// as an error on the host instead of a hung GPU.
//
// Counterparts in the reference: pipeline/src/comm.cu:58-114 (all-gather), :169-282 (reduce-scatter,
// fp16 adds), :284-323 (all-reduce = RS + AG in one kernel), :325-360 (all-reduce + RMSNorm),
// :475-485 (syncDevices); wrappers pipeline/include/netWrapper.cuh:141-402.
#include "common.cuh"
#include "kernels.h"
#include <string.h>

namespace nf {
namespace {

constexpr int kCommThreads = 256;
constexpr long long kPollLimitNs = 2000000000ll;

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_sys_v4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st_sys_v4(void* p, const uint4& v) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

// Bounded wait until *flag has reached `epoch` (wrap-safe). Returns false on timeout, and also as
// soon as the status word is set: once one wait of an iteration has run out (a peer is gone), the
// later collectives of that iteration give up at their first poll round instead of each spending its
// own two seconds, so a dead peer costs one time limit, not one per collective.
__device__ __forceinline__ bool wait_flag(const unsigned int* flag, unsigned int epoch,
                                          const unsigned int* status = nullptr) {
  uint64_t t0 = 0;
  for (unsigned int it = 0;; ++it) {
    if (static_cast<int>(ld_acquire_sys(flag) - epoch) >= 0) return true;
    if ((it & 63u) == 63u) {
      if (status != nullptr && *reinterpret_cast<const volatile unsigned int*>(status) != 0u) return false;
      uint64_t now;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
      if (t0 == 0) t0 = now;
      if (static_cast<long long>(now - t0) > kPollLimitNs) return false;
      __nanosleep(100);
    }
  }
}

struct FlagBlock {          // one per collective op instance, at the same heap offset on all ranks
  unsigned int ready[8];    // ready[src]: rank src's input is complete
  unsigned int done[8];     // done[src]: rank src has finished pushing into this rank
  unsigned int cta_counter;
  unsigned int pad[15];
};

__device__ __forceinline__ FlagBlock* flags_of(const nfk_comm_ctx& c, int r, long long off) {
  return reinterpret_cast<FlagBlock*>(reinterpret_cast<char*>(c.heap[r]) + off);
}

// Entry handshake: tell every rank that this rank's input is complete, wait for everyone's.
__device__ __forceinline__ void comm_enter(const nfk_comm_ctx& c, long long flag_off, unsigned int epoch,
                                           unsigned int* status, bool signal = true) {
  if (signal && blockIdx.x == 0 && threadIdx.x < c.nranks)
    st_release_sys(&flags_of(c, threadIdx.x, flag_off)->ready[c.rank], epoch);
  if (threadIdx.x < c.nranks) {
    if (!wait_flag(&flags_of(c, c.rank, flag_off)->ready[threadIdx.x], epoch, status))
      report_status(status, NF_ST_TIMEOUT_PEER_FLAG);
  }
  __syncthreads();
}

// Exit handshake: the last CTA of this rank tells every rank that its pushes have landed, then
// waits until every rank has said so, so the buffer is complete when the kernel ends.
__device__ __forceinline__ void comm_exit(const nfk_comm_ctx& c, long long flag_off, unsigned int epoch,
                                          unsigned int* status) {
  __shared__ int is_last;
  __threadfence_system();
  __syncthreads();
  FlagBlock* mine = flags_of(c, c.rank, flag_off);
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(&mine->cta_counter, 1u);
    is_last = (prev == gridDim.x - 1);
    if (is_last) mine->cta_counter = 0;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence_system();
  if (threadIdx.x < c.nranks) {
    st_release_sys(&flags_of(c, threadIdx.x, flag_off)->done[c.rank], epoch);
    if (!wait_flag(&mine->done[threadIdx.x], epoch, status)) report_status(status, NF_ST_TIMEOUT_PEER_FLAG);
  }
}

__device__ __forceinline__ float block_sum_comm(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < (kCommThreads >> 5)) ? red[lane] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

constexpr int kArThreads = 128;
constexpr int kGateRows = 128;       // rows per gate flag block (one M tile of the consumer GEMM)

// Owned rows (k indices: row = rank + nranks * k) of this rank inside gate block b of a `rows`-row buffer.
__device__ __forceinline__ int gate_owned_in_block(int b, int rows, int rank, int nranks) {
  const int lo_row = b * kGateRows, hi_row = min(rows, lo_row + kGateRows);
  const int lo = lo_row <= rank ? 0 : (lo_row - rank + nranks - 1) / nranks;
  const int hi = hi_row <= rank ? 0 : (hi_row - rank + nranks - 1) / nranks;
  return hi > lo ? hi - lo : 0;
}
__device__ __forceinline__ void gate_publish(const nfk_allreduce_params& p, int b) {
  for (int r = 0; r < p.ctx.nranks; ++r) {
    unsigned int* f = reinterpret_cast<unsigned int*>(reinterpret_cast<char*>(p.ctx.heap[r]) + p.gate_off) +
                      static_cast<long long>(b) * 8 + p.ctx.rank;
    st_release_sys(f, static_cast<unsigned int>(p.epoch));
  }
}
// Blocks in which this rank owns no row have nothing to wait for: publish them up front (one CTA).
__device__ __forceinline__ void gate_publish_empty_blocks(const nfk_allreduce_params& p) {
  if (p.gate_cnt == nullptr || blockIdx.x != 0) return;
  const int blocks = (p.rows + kGateRows - 1) / kGateRows;
  for (int b = threadIdx.x; b < blocks; b += blockDim.x)
    if (gate_owned_in_block(b, p.rows, p.ctx.rank, p.ctx.nranks) == 0) gate_publish(p, b);
}
// Called by the whole CTA after it has pushed the normed row `row`: the CTA that completes this rank's
// share of the row's block tells every rank. The system-scope fence of every thread orders its pushes
// before the count; the publishing thread's release store orders the counts it has seen before the flag.
__device__ __forceinline__ void gate_row_done(const nfk_allreduce_params& p, long long row) {
  if (p.gate_cnt == nullptr) return;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int b = static_cast<int>(row / kGateRows);
    const unsigned int want = static_cast<unsigned int>(gate_owned_in_block(b, p.rows, p.ctx.rank, p.ctx.nranks));
    const unsigned int prev = atomicAdd(&p.gate_cnt[b], 1u);
    if (prev + 1 == want) {
      p.gate_cnt[b] = 0;
      __threadfence_system();
      gate_publish(p, b);
    }
  }
}
constexpr int kArVec = 8;                                  // 16-byte vectors per thread per row
constexpr int kMaxCols = kArVec * 8 * kArThreads;          // 8192 columns

__device__ __forceinline__ float block_sum_ar(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < (kArThreads >> 5)) ? red[lane] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

// Small CTAs (128 threads, <= 168 registers, no dynamic shared memory) so that they fit on an SM
// next to a resident GEMM CTA: the collective then runs beside the GEMMs of another nano-batch
// instead of waiting for SMs. Loads over NVLink have microseconds of latency, so each thread keeps
// 16 independent 16-byte loads in flight (CH vectors x NR ranks) before it reduces and pushes.
//
// WIDE doubles the loads a thread has in flight per phase (32 instead of 16; used with 8 ranks), which
// halves the number of dependent load phases per row. The registers come from not keeping the summed
// row for the norm pass: the thread reads its own stores back (from sum_out, or from its own copy of
// the buffer when the sum is pushed), which are in L2.
template <int NR, bool NORM, bool WIDE>
__global__ void __launch_bounds__(kArThreads, 3)
allreduce_kernel(nfk_allreduce_params p) {
  constexpr int CH0 = NR >= 8 ? 2 : (NR >= 4 ? 4 : 8);    // vectors per chunk
  constexpr int CH = (WIDE && CH0 < 8) ? 2 * CH0 : CH0;
  constexpr bool REREAD = WIDE && NORM;
  __shared__ float red[8];
  const nfk_comm_ctx& c = p.ctx;
  // src_mode 1: the producer GEMM pushed the partial rows into local slabs and raised the ready flags
  comm_enter(c, p.flag_off, static_cast<unsigned int>(p.epoch), p.status, p.src_mode != 1);
  gate_publish_empty_blocks(p);

  const int nvec = p.cols >> 3;
  const long long row_bytes = p.ld * 2;
  const uint4* wv = NORM ? reinterpret_cast<const uint4*>(p.norm_w) : nullptr;
  const char* local_base = reinterpret_cast<const char*>(c.heap[c.rank]) + p.buf_off;
  const char* resid = reinterpret_cast<const char*>(p.resid);
  char* sum_out = reinterpret_cast<char*>(p.sum_out);
  const int owned = (p.rows - c.rank + NR - 1) / NR;       // rows rank, rank+NR, ... (may be <= 0)
  for (int k = blockIdx.x; k < owned; k += gridDim.x) {
    const long long row = c.rank + static_cast<long long>(NR) * k;
    uint4 packed[REREAD ? 1 : kArVec];
    float ss = 0.f;
#pragma unroll
    for (int i0 = 0; i0 < kArVec; i0 += CH) {
      uint4 in[CH][NR];
      uint4 rs[CH];
#pragma unroll
      for (int i = 0; i < CH; ++i) {
        const int v = threadIdx.x + (i0 + i) * kArThreads;
        if (v < nvec) {
          if (p.src_mode == 0) {
#pragma unroll
            for (int r = 0; r < NR; ++r)
              in[i][r] = ld_sys_v4(reinterpret_cast<const char*>(c.heap[r]) + p.buf_off + row * row_bytes + v * 16);
          } else if (p.src_mode == 2) {
            // column blocks: rank r produced columns [r * cols / NR, (r + 1) * cols / NR) of every row (an
            // N-split GEMM), so the row is gathered, one load per vector, instead of summed
            const int src = (v << 3) / (p.cols / NR);
            const char* base = reinterpret_cast<const char*>(c.heap[0]);
#pragma unroll
            for (int r = 1; r < NR; ++r)      // a chain of selects: no indexed read of the parameter block
              if (r == src) base = reinterpret_cast<const char*>(c.heap[r]);
            in[i][0] = ld_sys_v4(base + p.buf_off + row * row_bytes + v * 16);
#pragma unroll
            for (int r = 1; r < NR; ++r) in[i][r] = make_uint4(0u, 0u, 0u, 0u);
          } else {
#pragma unroll
            for (int r = 0; r < NR; ++r)
              in[i][r] = ld_sys_v4(local_base + (static_cast<long long>(r) * p.slab_rows + k) * row_bytes + v * 16);
          }
          if (resid != nullptr) rs[i] = *reinterpret_cast<const uint4*>(resid + row * p.resid_ld * 2 + v * 16);
        }
      }
#pragma unroll
      for (int i = 0; i < CH; ++i) {
        const int v = threadIdx.x + (i0 + i) * kArThreads;
        if (v < nvec) {
          float acc[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[e] = 0.f;
          if (resid != nullptr) {
            const uint32_t w4[4] = {rs[i].x, rs[i].y, rs[i].z, rs[i].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f = unpack_bf16x2(w4[e]);
              acc[2 * e] = f.x;
              acc[2 * e + 1] = f.y;
            }
          }
#pragma unroll
          for (int r = 0; r < NR; ++r) {
            const uint32_t w4[4] = {in[i][r].x, in[i][r].y, in[i][r].z, in[i][r].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f = unpack_bf16x2(w4[e]);
              acc[2 * e] += f.x;
              acc[2 * e + 1] += f.y;
            }
          }
          uint4 o;
          o.x = pack_bf16x2(acc[0], acc[1]);
          o.y = pack_bf16x2(acc[2], acc[3]);
          o.z = pack_bf16x2(acc[4], acc[5]);
          o.w = pack_bf16x2(acc[6], acc[7]);
          if (!REREAD) packed[i0 + i] = o;
          if (sum_out != nullptr) *reinterpret_cast<uint4*>(sum_out + row * p.sum_ld * 2 + v * 16) = o;
          if (p.push_sum) {
#pragma unroll
            for (int r = 0; r < NR; ++r)
              st_sys_v4(reinterpret_cast<char*>(c.heap[r]) + p.buf_off + row * row_bytes + v * 16, o);
          }
          if (NORM) {
            // normalise what was stored (bf16-rounded), as the standalone norm kernel would read it
            const uint32_t ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f = unpack_bf16x2(ow[e]);
              ss += f.x * f.x + f.y * f.y;
            }
          }
        }
      }
    }
    if (NORM) {
      const float tot = block_sum_ar(ss, red);
      const float inv = rsqrtf(tot / static_cast<float>(p.cols) + p.eps);
#pragma unroll
      for (int i = 0; i < kArVec; ++i) {
        const int v = threadIdx.x + i * kArThreads;
        if (v < nvec) {
          const uint4 ww = wv[v];
          const uint32_t w4[4] = {ww.x, ww.y, ww.z, ww.w};
          uint4 xs;
          if (REREAD) {
            // this thread's own store of the summed vector, a few microseconds old
            xs = sum_out != nullptr
                     ? *reinterpret_cast<const uint4*>(sum_out + row * p.sum_ld * 2 + v * 16)
                     : ld_sys_v4(reinterpret_cast<const char*>(c.heap[c.rank]) + p.buf_off + row * row_bytes + v * 16);
          } else {
            xs = packed[i];
          }
          const uint32_t x4[4] = {xs.x, xs.y, xs.z, xs.w};
          uint32_t ov[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 g = unpack_bf16x2(w4[e]);
            const float2 f = unpack_bf16x2(x4[e]);
            ov[e] = pack_bf16x2(f.x * inv * g.x, f.y * inv * g.y);
          }
          const uint4 o = make_uint4(ov[0], ov[1], ov[2], ov[3]);
          if (p.push_mode == 1) {
            *reinterpret_cast<uint4*>(reinterpret_cast<char*>(c.heap[c.rank]) + p.norm_out_off +
                                      row * static_cast<long long>(p.norm_ld) * 2 + v * 16) = o;
          } else {
#pragma unroll
            for (int r = 0; r < NR; ++r)
              st_sys_v4(reinterpret_cast<char*>(c.heap[r]) + p.norm_out_off +
                            row * static_cast<long long>(p.norm_ld) * 2 + v * 16, o);
          }
        }
      }
      gate_row_done(p, row);
    }
  }
  if (p.push_mode == 1) return;     // the caller's copies and barrier follow on the stream
  comm_exit(c, p.flag_off, static_cast<unsigned int>(p.epoch), p.status);
}

// ---- in-switch (NVLS) form -------------------------------------------------------------------------
// With the heaps bound to one NVLink multicast object, a load from the multicast address of a word is
// answered by the NVSwitch with the sum of that word over all ranks (multimem.ld_reduce, bf16 inputs
// added in fp32), and a store to it lands in every rank's copy (multimem.st). The owner of a row then
// needs one 16-byte load per 8 columns instead of one per rank, and one store instead of one per rank:
// an eighth of the instructions in flight for the same bytes of result, and about two thirds of the bytes
// on this GPU's links (its own partial rows still leave once, the normed rows of the others still arrive).
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_v4(void* mc, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

// One row per CTA pass with the whole row in flight at once (8 multimem loads + 8 residual loads per
// thread), and the next row's loads issued before the current row is summed, normalised and stored, so
// that a CTA always has a row on the wire; rows r, r + nranks, ... of the buffer belong to rank r as in
// allreduce_kernel. The switch returns the ranks' sum already rounded to bf16; the residual is added to
// that in fp32 and the result rounded once more, so sums can differ from allreduce_kernel's (one
// rounding) in the last bf16 bit.
template <bool NORM>
__global__ void __launch_bounds__(kArThreads, 3)
allreduce_mc_kernel(nfk_allreduce_params p) {
  __shared__ float red[8];
  const nfk_comm_ctx& c = p.ctx;
  comm_enter(c, p.flag_off, static_cast<unsigned int>(p.epoch), p.status, true);
  gate_publish_empty_blocks(p);
  const int NR = c.nranks;
  const int nvec = p.cols >> 3;
  const long long row_bytes = p.ld * 2;
  const uint4* wv = NORM ? reinterpret_cast<const uint4*>(p.norm_w) : nullptr;
  char* mc = reinterpret_cast<char*>(p.mc_heap);
  const char* resid = reinterpret_cast<const char*>(p.resid);
  char* sum_out = reinterpret_cast<char*>(p.sum_out);
  const int owned = (p.rows - c.rank + NR - 1) / NR;
  uint4 in[kArVec], rs[kArVec], in_nx[kArVec], rs_nx[kArVec];
  auto fetch = [&](int k, uint4 (&a)[kArVec], uint4 (&b)[kArVec]) {
    const long long row = c.rank + static_cast<long long>(NR) * k;
#pragma unroll
    for (int i = 0; i < kArVec; ++i) {
      const int v = threadIdx.x + i * kArThreads;
      if (v < nvec) {
        a[i] = multimem_ld_reduce_bf16x8(mc + p.buf_off + row * row_bytes + v * 16);
        if (resid != nullptr) b[i] = *reinterpret_cast<const uint4*>(resid + row * p.resid_ld * 2 + v * 16);
      }
    }
  };
  int k = blockIdx.x;
  if (k < owned) fetch(k, in, rs);
  for (; k < owned; k += gridDim.x) {
    const long long row = c.rank + static_cast<long long>(NR) * k;
    const int k_next = k + gridDim.x;
    if (k_next < owned) fetch(k_next, in_nx, rs_nx);
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kArVec; ++i) {
      const int v = threadIdx.x + i * kArThreads;
      if (v < nvec) {
        uint4 o = in[i];
        if (resid != nullptr) {
          const uint32_t a4[4] = {in[i].x, in[i].y, in[i].z, in[i].w};
          const uint32_t b4[4] = {rs[i].x, rs[i].y, rs[i].z, rs[i].w};
          uint32_t o4[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 a = unpack_bf16x2(a4[e]), b = unpack_bf16x2(b4[e]);
            o4[e] = pack_bf16x2(a.x + b.x, a.y + b.y);
          }
          o = make_uint4(o4[0], o4[1], o4[2], o4[3]);
        }
        in[i] = o;
        if (sum_out != nullptr) *reinterpret_cast<uint4*>(sum_out + row * p.sum_ld * 2 + v * 16) = o;
        if (p.push_sum) multimem_st_v4(mc + p.buf_off + row * row_bytes + v * 16, o);
        if (NORM) {
          const uint32_t ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = unpack_bf16x2(ow[e]);
            ss += f.x * f.x + f.y * f.y;
          }
        }
      }
    }
    if (NORM) {
      const float tot = block_sum_ar(ss, red);
      const float inv = rsqrtf(tot / static_cast<float>(p.cols) + p.eps);
#pragma unroll
      for (int i = 0; i < kArVec; ++i) {
        const int v = threadIdx.x + i * kArThreads;
        if (v < nvec) {
          const uint4 ww = wv[v];
          const uint32_t w4[4] = {ww.x, ww.y, ww.z, ww.w};
          const uint32_t x4[4] = {in[i].x, in[i].y, in[i].z, in[i].w};
          uint32_t ov[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 g = unpack_bf16x2(w4[e]);
            const float2 f = unpack_bf16x2(x4[e]);
            ov[e] = pack_bf16x2(f.x * inv * g.x, f.y * inv * g.y);
          }
          const uint4 o = make_uint4(ov[0], ov[1], ov[2], ov[3]);
          if (p.push_mode == 1)
            *reinterpret_cast<uint4*>(reinterpret_cast<char*>(c.heap[c.rank]) + p.norm_out_off +
                                      row * static_cast<long long>(p.norm_ld) * 2 + v * 16) = o;
          else
            multimem_st_v4(mc + p.norm_out_off + row * static_cast<long long>(p.norm_ld) * 2 + v * 16, o);
        }
      }
      gate_row_done(p, row);
    }
#pragma unroll
    for (int i = 0; i < kArVec; ++i) {
      in[i] = in_nx[i];
      rs[i] = rs_nx[i];
    }
  }
  if (p.push_mode == 1) return;     // the caller's copies and barrier follow on the stream
  comm_exit(c, p.flag_off, static_cast<unsigned int>(p.epoch), p.status);
}

// A collective's CTAs are meant to share SMs with the CTAs of a GEMM that is launched after it. An SM
// changes its L1 / shared-memory split only while idle, so a kernel that asks for no shared memory
// would leave its SMs configured with too little for a GEMM CTA until it exits. Asking for the
// largest shared-memory split keeps those SMs open to GEMM CTAs.
template <typename K>
void prefer_max_shared(K kernel) {
  (void)cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  (void)cudaGetLastError();
}

template <int NR>
int launch_allreduce(const nfk_allreduce_params* p, int ctas, cudaStream_t stream) {
  static bool once_dev[kMaxDevices] = {false};   // the attribute is per device
  bool& once = once_dev[device_slot()];
  if (!once) {
    prefer_max_shared(allreduce_kernel<NR, true, false>);
    prefer_max_shared(allreduce_kernel<NR, false, false>);
    if constexpr (NR >= 8) {
      prefer_max_shared(allreduce_kernel<NR, true, true>);
      prefer_max_shared(allreduce_kernel<NR, false, true>);
    }
    once = true;
  }
  const bool norm = p->norm_w != nullptr;
  if (p->mc_heap != nullptr && p->src_mode == 0 && NR > 1) {
    static bool once_mc_dev[kMaxDevices] = {false};
    bool& once_mc = once_mc_dev[device_slot()];
    if (!once_mc) {
      prefer_max_shared(allreduce_mc_kernel<true>);
      prefer_max_shared(allreduce_mc_kernel<false>);
      once_mc = true;
    }
    if (norm)
      allreduce_mc_kernel<true><<<ctas, kArThreads, 0, stream>>>(*p);
    else
      allreduce_mc_kernel<false><<<ctas, kArThreads, 0, stream>>>(*p);
    return cudaGetLastError() == cudaSuccess ? NF_OK : NF_ERR_CUDA;
  }
  if constexpr (NR >= 8) {
    // The wide form with a norm reads the sum back, so the sum must have been stored somewhere local.
    if (p->wide != 0 && (!norm || p->sum_out != nullptr || p->push_sum != 0)) {
      if (norm)
        allreduce_kernel<NR, true, true><<<ctas, kArThreads, 0, stream>>>(*p);
      else
        allreduce_kernel<NR, false, true><<<ctas, kArThreads, 0, stream>>>(*p);
      return cudaGetLastError() == cudaSuccess ? NF_OK : NF_ERR_CUDA;
    }
  }
  if (norm)
    allreduce_kernel<NR, true, false><<<ctas, kArThreads, 0, stream>>>(*p);
  else
    allreduce_kernel<NR, false, false><<<ctas, kArThreads, 0, stream>>>(*p);
  return cudaGetLastError() == cudaSuccess ? NF_OK : NF_ERR_CUDA;
}

__global__ void __launch_bounds__(kCommThreads)
allgather_kernel(nfk_allgather_params p) {
  const nfk_comm_ctx& c = p.ctx;
  if (p.handshake_in) comm_enter(c, p.flag_off, static_cast<unsigned int>(p.epoch), p.status);
  const long long row_vec = p.shard_bytes >> 4;                  // 16-byte vectors of this rank's shard per row
  const long long rows = p.rows > 1 ? p.rows : 1;
  const long long nvec = row_vec * rows;
  const long long mine = p.buf_off + c.rank * p.shard_stride;    // same offset in every rank's heap
  const char* src = reinterpret_cast<const char*>(c.heap[c.rank]) + mine;
  for (long long v = blockIdx.x * static_cast<long long>(kCommThreads) + threadIdx.x; v < nvec;
       v += static_cast<long long>(gridDim.x) * kCommThreads) {
    const long long off = rows > 1 ? (v / row_vec) * p.row_stride + (v % row_vec) * 16 : v * 16;
    const uint4 val = *reinterpret_cast<const uint4*>(src + off);
#pragma unroll
    for (int r = 0; r < 8; ++r)
      if (r < c.nranks && r != c.rank) st_sys_v4(reinterpret_cast<char*>(c.heap[r]) + mine + off, val);
  }
  comm_exit(c, p.flag_off, static_cast<unsigned int>(p.epoch), p.status);
}

__global__ void comm_barrier_kernel(nfk_comm_ctx c, long long flag_off, int epoch, unsigned int* status) {
  if (threadIdx.x < c.nranks) {
    st_release_sys(&flags_of(c, threadIdx.x, flag_off)->ready[c.rank], static_cast<unsigned int>(epoch));
    if (!wait_flag(&flags_of(c, c.rank, flag_off)->ready[threadIdx.x], static_cast<unsigned int>(epoch), status))
      report_status(status, NF_ST_TIMEOUT_PEER_FLAG);
  }
}

bool ctx_ok(const nfk_comm_ctx& c) {
  if (c.nranks < 1 || c.nranks > 8 || c.rank < 0 || c.rank >= c.nranks) return false;
  for (int r = 0; r < c.nranks; ++r)
    if (c.heap[r] == nullptr) return false;
  return true;
}

}  // namespace
}  // namespace nf

extern "C" int nfk_allreduce(const nfk_allreduce_params* p, cudaStream_t stream) {
  using namespace nf;
  if (!p || !ctx_ok(p->ctx)) return NF_ERR_BAD_ARG;
  if (p->cols <= 0 || p->cols % 8 != 0 || p->cols > kMaxCols || p->ld % 8 != 0 || p->rows < 0 ||
      p->buf_off % 16 != 0 || p->flag_off % 16 != 0)
    return NF_ERR_BAD_ARG;
  if (p->norm_w != nullptr && (p->norm_out_off % 16 != 0 || p->norm_ld % 8 != 0)) return NF_ERR_BAD_ARG;
  if (p->resid != nullptr && ((reinterpret_cast<uintptr_t>(p->resid) & 15) || p->resid_ld % 8 != 0))
    return NF_ERR_BAD_ARG;
  if (p->sum_out != nullptr && ((reinterpret_cast<uintptr_t>(p->sum_out) & 15) || p->sum_ld % 8 != 0))
    return NF_ERR_BAD_ARG;
  if (p->src_mode == 1 && (p->push_sum != 0 || p->slab_rows * p->ctx.nranks < p->rows))
    return NF_ERR_BAD_ARG;   // slab input: the sum cannot be pushed back into a per-rank buffer
  if (p->src_mode == 2 && p->cols % (8 * p->ctx.nranks) != 0) return NF_ERR_BAD_ARG;   // whole vectors per block
  if (p->src_mode < 0 || p->src_mode > 2) return NF_ERR_BAD_ARG;
  if (p->mc_heap != nullptr && (reinterpret_cast<uintptr_t>(p->mc_heap) & 15) != 0) return NF_ERR_BAD_ARG;
  if (p->gate_cnt != nullptr && (p->norm_w == nullptr || p->gate_off % 16 != 0)) return NF_ERR_BAD_ARG;
  if (p->push_mode != 0 && (p->push_mode != 1 || p->norm_w == nullptr || p->gate_cnt != nullptr || p->push_sum != 0))
    return NF_ERR_BAD_ARG;
  // Even an empty buffer takes part in the handshakes so that all ranks stay in step.
  const int nr = p->ctx.nranks;
  const int owned = (p->rows + nr - 1) / nr;
  int ctas = p->num_ctas > 0 ? p->num_ctas : device_sm_count();
  if (ctas > owned) ctas = owned > 0 ? owned : 1;
  switch (nr) {
    case 1: return launch_allreduce<1>(p, ctas, stream);
    case 2: return launch_allreduce<2>(p, ctas, stream);
    case 4: return launch_allreduce<4>(p, ctas, stream);
    case 8: return launch_allreduce<8>(p, ctas, stream);
    default: return NF_ERR_UNSUPPORTED;
  }
}

extern "C" int nfk_allgather(const nfk_allgather_params* p, cudaStream_t stream) {
  using namespace nf;
  if (!p || !ctx_ok(p->ctx)) return NF_ERR_BAD_ARG;
  if (p->shard_bytes < 0 || p->shard_bytes % 16 != 0 || p->shard_stride % 16 != 0 || p->buf_off % 16 != 0 ||
      p->flag_off % 16 != 0 || p->shard_stride < p->shard_bytes)
    return NF_ERR_BAD_ARG;
  if (p->rows < 0 || (p->rows > 1 && (p->row_stride % 16 != 0 || p->row_stride < p->ctx.nranks * p->shard_stride)))
    return NF_ERR_BAD_ARG;
  long long ctas = p->num_ctas > 0 ? p->num_ctas : 16;
  const long long need = ((p->shard_bytes >> 4) * (p->rows > 1 ? p->rows : 1) + kCommThreads - 1) / kCommThreads;
  if (ctas > need) ctas = need > 0 ? need : 1;
  static bool once_dev[kMaxDevices] = {false};   // the attribute is per device
  bool& once = once_dev[device_slot()];
  if (!once) {
    prefer_max_shared(allgather_kernel);
    once = true;
  }
  allgather_kernel<<<static_cast<int>(ctas), kCommThreads, 0, stream>>>(*p);
  return cudaGetLastError() == cudaSuccess ? NF_OK : NF_ERR_CUDA;
}

extern "C" int nfk_comm_barrier(const nfk_comm_barrier_params* p, cudaStream_t stream) {
  using namespace nf;
  if (!p || !ctx_ok(p->ctx) || p->flag_off % 16 != 0) return NF_ERR_BAD_ARG;
  static bool once_dev[kMaxDevices] = {false};   // the attribute is per device
  bool& once = once_dev[device_slot()];
  if (!once) {
    prefer_max_shared(comm_barrier_kernel);
    once = true;
  }
  comm_barrier_kernel<<<1, 32, 0, stream>>>(p->ctx, p->flag_off, p->epoch, p->status);
  return cudaGetLastError() == cudaSuccess ? NF_OK : NF_ERR_CUDA;
}

// ---- symmetric heap plumbing (host) -----------------------------------------------------------------
extern "C" int nfk_symm_alloc(void** out, long long bytes) {
  using namespace nf;
  if (!out || bytes <= 0) return NF_ERR_BAD_ARG;
  if (cudaMalloc(out, static_cast<size_t>(bytes)) != cudaSuccess) return NF_ERR_CUDA;
  if (cudaMemset(*out, 0, static_cast<size_t>(bytes)) != cudaSuccess) return NF_ERR_CUDA;
  return cudaDeviceSynchronize() == cudaSuccess ? NF_OK : NF_ERR_CUDA;
}
extern "C" int nfk_symm_free(void* p) { return cudaFree(p) == cudaSuccess ? nf::NF_OK : nf::NF_ERR_CUDA; }
extern "C" int nfk_ipc_get_handle(void* ptr, unsigned char* out64) {
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, ptr) != cudaSuccess) return nf::NF_ERR_CUDA;
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(out64, &h, 64);
  return nf::NF_OK;
}
extern "C" int nfk_ipc_open_handle(const unsigned char* in64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, in64, 64);
  return cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess ? nf::NF_OK
                                                                                    : nf::NF_ERR_CUDA;
}
extern "C" int nfk_ipc_close_handle(void* p) {
  return cudaIpcCloseMemHandle(p) == cudaSuccess ? nf::NF_OK : nf::NF_ERR_CUDA;
}
