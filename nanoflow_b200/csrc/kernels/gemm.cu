// bf16 GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM), operands staged
// by TMA into 128B-swizzled shared memory, persistent over output tiles with an explicit CTA budget.
//
//   D[M,N] = A[M,K] * B[N,K]^T (+ bias[N]) (+ beta * C[M,N])            (linear epilogue)
//   D[M,F] = silu(A * Bg[F,K]^T) .* (A * Bu[F,K]^T)                      (SwiGLU epilogue)
//
// Roles inside one 192-thread CTA: warp 0 lane 0 = TMA producer, warp 1 = TMEM owner and (lane 0)
// MMA issuer, warps 2..5 = epilogue (TMEM -> registers -> global). Two TMEM accumulators are
// ping-ponged so the epilogue of tile i overlaps the main loop of tile i+1.
//
// Takes the place of the reference's CUTLASS Sm80 device::Gemm wrapper
// (pipeline/include/cutlassGemmWrapperImpl.cuh:68-125: D = alpha*A*B + beta*C, residual or
// replicated bias as C) and of its DualGemm + SiLU-mul epilogue (pipeline/include/dualWrapper.cuh:47-144).
#include "common.cuh"
#include "kernels.h"

#include <mutex>

namespace nf {

nf_encode_tiled_fn get_encode_tiled() {
  static nf_encode_tiled_fn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<nf_encode_tiled_fn>(p);
    }
  });
  return fn;
}

int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols,
                      uint64_t ld, uint32_t box_rows, uint32_t box_cols) {
  nf_encode_tiled_fn enc = get_encode_tiled();
  if (enc == nullptr) return NF_ERR_CUDA;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (ld * 2) % 16 != 0) return NF_ERR_BAD_ARG;
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim, gstride,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? NF_OK : NF_ERR_CUDA;
}

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kGemmThreads = 192;

template <int BN>
struct Cfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
};

struct DevParams {
  __nv_bfloat16* D;
  const __nv_bfloat16* C;
  const __nv_bfloat16* bias;
  long long ldd, ldc;
  float beta;
  int M, N, K;  // N = number of output columns
  unsigned int* status;
};

// Wait helper shared by all roles: bounded by wall clock (globaltimer) and by the CTA abort flag.
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  const uint32_t addr = smem_u32(bar);
  uint64_t t0 = 0;
  for (uint32_t it = 0;; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(addr), "r"(parity)
        : "memory");
    if (ok) return true;
    if ((it & 255u) == 255u) {
      if (*abort_flag) return false;
      uint64_t now;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
      if (t0 == 0) t0 = now;
      if (now - t0 > 2000000000ull || it > (1u << 30)) return false;  // 2 s
    }
  }
}

template <int BN, int EPI>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB0,
                    const __grid_constant__ CUtensorMap tmB1, DevParams p) {
  using C = Cfg<BN>;
  constexpr int STAGES = C::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * C::STAGE_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tmem_full = bars + 2 * STAGES;
  uint64_t* tmem_empty = bars + 2 * STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // Output tile width: the SwiGLU epilogue folds a gate half and an up half of BN/2 columns each.
  constexpr int OUT_BN = (EPI == 1) ? BN / 2 : BN;
  const int m_blocks = (p.M + BM - 1) / BM;
  const int n_blocks = (p.N + OUT_BN - 1) / OUT_BN;
  const int num_tiles = m_blocks * n_blocks;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB0);
    if (EPI == 1) tma_prefetch_desc(&tmB1);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0 && lane == 0) {
    // ---------------- TMA producer ----------------
    uint32_t it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const int m_blk = tile % m_blocks;
      const int n_blk = tile / m_blocks;
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!wait_or_abort(&empty_bar[s], ph ^ 1, abort_flag)) {
          report_status(p.status, NF_ST_TIMEOUT_SMEM_EMPTY);
          *abort_flag = 1;
          ok = false;
          break;
        }
        uint8_t* sa = smem + s * C::STAGE_BYTES;
        uint8_t* sb = sa + C::A_BYTES;
        mbar_expect_tx(&full_bar[s], C::STAGE_BYTES);
        tma_load_2d(sa, &tmA, &full_bar[s], kb * BK, m_blk * BM);
        if (EPI == 1) {
          tma_load_2d(sb, &tmB0, &full_bar[s], kb * BK, n_blk * OUT_BN);
          tma_load_2d(sb + C::B_BYTES / 2, &tmB1, &full_bar[s], kb * BK, n_blk * OUT_BN);
        } else {
          tma_load_2d(sb, &tmB0, &full_bar[s], kb * BK, n_blk * BN);
        }
      }
    }
    if (!ok) {
      // Drain: give loads already in flight a bounded chance to land before the CTA exits.
      const uint32_t issued = it;
      const uint32_t back = issued < static_cast<uint32_t>(STAGES) ? issued : STAGES;
      for (uint32_t j = issued - back; j < issued; ++j) {
        const int s = j % STAGES;
        const uint32_t ph = (j / STAGES) & 1;
        for (int spin = 0; spin < 100000; ++spin) {
          uint32_t done;
          asm volatile(
              "{\n\t.reg .pred p;\n\t"
              "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
              "selp.u32 %0, 1, 0, p;\n\t}"
              : "=r"(done)
              : "r"(smem_u32(&full_bar[s])), "r"(ph)
              : "memory");
          if (done) break;
        }
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------- MMA issuer ----------------
    constexpr uint32_t idesc = umma_idesc_bf16(BM, BN);
    uint32_t it = 0, tcount = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tcount) {
      const uint32_t acc = tcount & 1;
      const uint32_t acc_ph = (tcount >> 1) & 1;
      if (!wait_or_abort(&tmem_empty[acc], acc_ph ^ 1, abort_flag)) {
        report_status(p.status, NF_ST_TIMEOUT_TMEM_EMPTY);
        *abort_flag = 1;
        break;
      }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * BN;
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!wait_or_abort(&full_bar[s], ph, abort_flag)) {
          report_status(p.status, NF_ST_TIMEOUT_SMEM_FULL);
          *abort_flag = 1;
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smem + s * C::STAGE_BYTES);
        const uint32_t b_addr = a_addr + C::A_BYTES;
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          const uint64_t da = umma_desc_k_sw128(a_addr + k * UMMA_K * 2);
          const uint64_t db = umma_desc_k_sw128(b_addr + k * UMMA_K * 2);
          umma_bf16_ss(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
        }
        umma_commit(&empty_bar[s]);  // stage is free once these MMAs have read it
      }
      if (ok) umma_commit(&tmem_full[acc]);
    }
  } else if (warp >= 2) {
    // ---------------- epilogue ----------------
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    uint32_t tcount = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++tcount) {
      const int m_blk = tile % m_blocks;
      const int n_blk = tile / m_blocks;
      const uint32_t acc = tcount & 1;
      const uint32_t acc_ph = (tcount >> 1) & 1;
      if (!wait_or_abort(&tmem_full[acc], acc_ph, abort_flag)) {
        if (lane == 0) report_status(p.status, NF_ST_TIMEOUT_TMEM_FULL);
        *abort_flag = 1;
        break;
      }
      __syncwarp();
      tc_fence_after();
      const int row = m_blk * BM + q * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      __nv_bfloat16* drow = p.D + static_cast<long long>(row) * p.ldd;
      const __nv_bfloat16* crow =
          (EPI == 0 && p.C != nullptr) ? p.C + static_cast<long long>(row) * p.ldc : nullptr;
#pragma unroll 1
      for (int c = 0; c < OUT_BN / 32; ++c) {
        uint32_t r[32];
        float v[32];
        tmem_ld_32x32b_x32(t_row + c * 32, r);
        if (EPI == 1) {
          uint32_t u[32];
          tmem_ld_32x32b_x32(t_row + BN / 2 + c * 32, u);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float g = __uint_as_float(r[j]);
            const float up = __uint_as_float(u[j]);
            v[j] = g / (1.0f + __expf(-g)) * up;
          }
        } else {
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        }
        const int col0 = n_blk * OUT_BN + c * 32;
        if (row_ok && col0 < p.N) {
#pragma unroll
          for (int g8 = 0; g8 < 4; ++g8) {
            const int col = col0 + g8 * 8;
            if (col < p.N) {  // N is a multiple of 8
              float* vv = v + g8 * 8;
              if (EPI == 0) {
                if (p.bias != nullptr) {
                  const uint4 bv = *reinterpret_cast<const uint4*>(p.bias + col);
                  const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    const float2 f = unpack_bf16x2(bw[j]);
                    vv[2 * j] += f.x;
                    vv[2 * j + 1] += f.y;
                  }
                }
                if (crow != nullptr) {
                  const uint4 cv = *reinterpret_cast<const uint4*>(crow + col);
                  const uint32_t cw[4] = {cv.x, cv.y, cv.z, cv.w};
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    const float2 f = unpack_bf16x2(cw[j]);
                    vv[2 * j] += p.beta * f.x;
                    vv[2 * j + 1] += p.beta * f.y;
                  }
                }
              }
              uint4 o;
              o.x = pack_bf16x2(vv[0], vv[1]);
              o.y = pack_bf16x2(vv[2], vv[3]);
              o.z = pack_bf16x2(vv[4], vv[5]);
              o.w = pack_bf16x2(vv[6], vv[7]);
              *reinterpret_cast<uint4*>(drow + col) = o;
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

template <int BN, int EPI>
int launch(const nfk_gemm_params& g, cudaStream_t stream) {
  using C = Cfg<BN>;
  constexpr int OUT_BN = (EPI == 1) ? BN / 2 : BN;
  CUtensorMap tmA, tmB0, tmB1;
  int rc = make_tmap_bf16_2d(&tmA, g.A, g.M, g.K, g.lda, BM, BK);
  if (rc != NF_OK) return rc;
  rc = make_tmap_bf16_2d(&tmB0, g.B, g.N, g.K, g.ldb, OUT_BN, BK);
  if (rc != NF_OK) return rc;
  if (EPI == 1) {
    rc = make_tmap_bf16_2d(&tmB1, g.B2, g.N, g.K, g.ldb, OUT_BN, BK);
    if (rc != NF_OK) return rc;
  } else {
    tmB1 = tmB0;
  }
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, EPI>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                             C::SMEM_BYTES) != cudaSuccess)
      return NF_ERR_CUDA;
    attr_set = true;
  }
  const int m_blocks = (g.M + BM - 1) / BM;
  const int n_blocks = (g.N + OUT_BN - 1) / OUT_BN;
  const int tiles = m_blocks * n_blocks;
  int ctas = g.num_ctas > 0 ? g.num_ctas : sm_count();
  if (ctas > tiles) ctas = tiles;
  DevParams p;
  p.D = reinterpret_cast<__nv_bfloat16*>(g.D);
  p.C = reinterpret_cast<const __nv_bfloat16*>(g.C);
  p.bias = reinterpret_cast<const __nv_bfloat16*>(g.bias);
  p.ldd = g.ldd;
  p.ldc = g.ldc;
  p.beta = g.beta;
  p.M = g.M;
  p.N = g.N;
  p.K = g.K;
  p.status = g.status;
  gemm_tcgen05_kernel<BN, EPI><<<ctas, kGemmThreads, C::SMEM_BYTES, stream>>>(tmA, tmB0, tmB1, p);
  return cudaGetLastError() == cudaSuccess ? NF_OK : NF_ERR_CUDA;
}

}  // namespace
}  // namespace nf

extern "C" int nfk_gemm_bf16(const nfk_gemm_params* g, cudaStream_t stream) {
  using namespace nf;
  if (g == nullptr) return NF_ERR_BAD_ARG;
  if (g->M == 0 || g->N == 0) return NF_OK;  // empty nano-batch: nothing to do
  if (g->A == nullptr || g->B == nullptr || g->D == nullptr) return NF_ERR_BAD_ARG;
  if (g->M < 0 || g->N < 0 || g->K <= 0) return NF_ERR_BAD_ARG;
  if (g->K % 8 != 0 || g->N % 8 != 0 || g->lda % 8 != 0 || g->ldb % 8 != 0 || g->ldd % 8 != 0)
    return NF_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(g->D) & 15) != 0) return NF_ERR_BAD_ARG;
  if (g->C != nullptr && ((reinterpret_cast<uintptr_t>(g->C) & 15) != 0 || g->ldc % 8 != 0))
    return NF_ERR_BAD_ARG;
  if (g->epilogue == NFK_EPI_SWIGLU) {
    if (g->B2 == nullptr) return NF_ERR_BAD_ARG;
    switch (g->tile_n) {
      case 0:
      case 256: return launch<256, 1>(*g, stream);
      case 128: return launch<128, 1>(*g, stream);
      default: return NF_ERR_UNSUPPORTED;
    }
  }
  int bn = g->tile_n;
  if (bn == 0) {
    // Pick the widest tile that still gives every SM of the budget a tile.
    const int ctas = g->num_ctas > 0 ? g->num_ctas : sm_count();
    const int m_blocks = (g->M + BM - 1) / BM;
    bn = 256;
    while (bn > 64 && m_blocks * ((g->N + bn - 1) / bn) < ctas) bn >>= 1;
  }
  switch (bn) {
    case 256: return launch<256, 0>(*g, stream);
    case 128: return launch<128, 0>(*g, stream);
    case 64: return launch<64, 0>(*g, stream);
    default: return NF_ERR_UNSUPPORTED;
  }
}
