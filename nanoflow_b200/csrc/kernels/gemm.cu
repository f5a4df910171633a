// bf16 GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM), operands staged
// by TMA into 128B-swizzled shared memory, persistent over output tiles with an explicit CTA budget.
//
//   D[M,N] = A[M,K] * B[N,K]^T (+ bias[N]) (+ beta * C[M,N])            (linear epilogue)
//   D[M,F] = silu(A * Bg[F,K]^T) .* (A * Bu[F,K]^T)                      (SwiGLU epilogue)
//
// Work units are whole output tiles, or with split-K (tile, k range) pairs whose fp32 partial tiles
// a second pass adds up; with the stream-K tail only the tiles left over after the full waves are
// cut, into equal k ranges. For small M one CTA can cover several M tiles with the same weight tile,
// so each weight byte is fetched into shared memory once; for larger M the two CTAs of a cluster
// share a 256-row tile (tcgen05.mma.cta_group::2) and each stages half of the weight tile. A cost
// model picks the shape; engines time the candidates on their own shapes (ops/autotune.py).
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

int device_slot() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  return (dev >= 0 && dev < kMaxDevices) ? dev : 0;
}

int device_sm_count() {
  static int cached[kMaxDevices] = {0};
  const int slot = device_slot();
  int n = cached[slot];
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, slot) != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      return 148;
    }
    cached[slot] = n;   // the same value from whichever thread gets here first
  }
  return n;
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
constexpr int kSmemBudget = 227 * 1024 - 2048;

// Tile geometry. The tile is 128*MT rows by `bn` weight rows (bn: multiple of 32 up to 256, a runtime
// value so that the tile count can be matched to the SM count); MT = number of 128-row M tiles one
// CTA covers with the same B tile (MT > 1 is the small-M, weight-streaming shape: every weight byte
// enters shared memory once). Shared memory: 1 KB of barriers, then `stages` ring slots of
// (MT*16 KB of A + bn*128 B of B). TMEM: MT*bn fp32 columns per accumulator set, two sets
// (epilogue of one tile under the main loop of the next) when they fit in 512 columns.
constexpr int kMaxStages = 8;
constexpr int A_TILE_BYTES = BM * BK * 2;
struct Geom {
  int bn, out_bn, stages, acc_bufs, tmem_cols, stage_bytes, b_bytes, smem_bytes;
};
// Reduce-scatter epilogue, staged form: each epilogue warp keeps a [32 rows][128 columns] bf16 piece of
// its rows in shared memory (row pitch 272 B, so that the 32 lanes' 16-byte stores spread over all
// banks) and sends each row's 256 bytes to its owner with one bulk copy.
constexpr int kRsRunCols = 128;
constexpr int kRsRowPitch = kRsRunCols * 2 + 16;
constexpr int kRsStageBytes = 4 * 32 * kRsRowPitch;     // four epilogue warps

inline Geom make_geom(int bn, int mt, bool swiglu, int smem_budget, int cg, int extra = 0) {
  Geom g;
  g.bn = bn;
  g.out_bn = swiglu ? bn / 2 : bn;
  g.b_bytes = (bn / cg) * BK * 2;      // a CTA pair splits the weight tile between its two CTAs
  g.stage_bytes = mt * A_TILE_BYTES + g.b_bytes;
  int st = (smem_budget - 2048 - extra) / g.stage_bytes;
  g.stages = st > kMaxStages ? kMaxStages : st;
  const int acc_cols = mt * bn;
  g.acc_bufs = acc_cols * 2 <= 512 ? 2 : 1;
  const int need = acc_cols * g.acc_bufs;
  g.tmem_cols = need <= 32 ? 32 : need <= 64 ? 64 : need <= 128 ? 128 : need <= 256 ? 256 : 512;
  g.smem_bytes = g.stages * g.stage_bytes + 2048 + extra;   // the extra region follows the ring slots
  return g;
}

struct DevParams {
  __nv_bfloat16* D;
  const __nv_bfloat16* C;
  const __nv_bfloat16* bias;
  float* partial;   // split-K: fp32 [split_k][M][N] partial sums (second pass reduces them)
  long long ldd, ldc;
  float beta;
  int M, N, K;      // N = number of output columns
  int split_k;
  unsigned int* status;
  int bn, stages, acc_bufs, tmem_cols;   // tile geometry (see make_geom)
  // stream-K tail (see Walk): tiles from sk_tiles_dp on are cut into k-block ranges of sk_q
  float* sk_partial;          // fp32 [tile][piece][CTA of pair][rows per CTA][bn]
  int sk_tiles_dp, sk_q, sk_max_pieces;
  // RMSNorm of the result rows, fused into the split-K reduce pass
  const __nv_bfloat16* norm_w;
  __nv_bfloat16* norm_out;
  long long norm_ld;
  float norm_eps;
  // reduce-scatter epilogue (EPI == 2)
  char* rs_heap[8];
  int rs_rank, rs_nranks, rs_rows_cap, rs_epoch;
  long long rs_slab_off, rs_flag_off;
  int rs_staged;     // partial rows leave through shared memory and bulk copies instead of 16-byte stores
  // gated input: see nfk_gemm_params::gate_flags
  const unsigned int* gate_flags;
  int gate_epoch, gate_nranks;
};

// Tile index -> (m group, n block). Normally m groups vary fastest, so CTAs that run together share
// weight panels in L2; with a gated input n blocks vary fastest, so the first wave of tiles needs only the
// first rows of A.
__device__ __forceinline__ void tile_coords(const DevParams& p, int tile, int m_groups, int n_blocks, int& m_grp,
                                            int& n_blk) {
  if (p.gate_flags != nullptr) {
    m_grp = tile / n_blocks;
    n_blk = tile - m_grp * n_blocks;
  } else {
    m_grp = tile % m_groups;
    n_blk = tile / m_groups;
  }
}

// Bounded wait until every rank has delivered its rows of 128-row block `m_tile` of A. The flags are
// written by remote stores (st.release.sys); the loads that follow are TMA copies (async proxy), hence
// the proxy fence after the acquire.
__device__ __forceinline__ bool wait_gate(const DevParams& p, int m_tile, volatile int* abort_flag) {
  const unsigned int* f = p.gate_flags + static_cast<long long>(m_tile) * 8;
  uint64_t t0 = 0;
  for (int r = 0; r < p.gate_nranks; ++r) {
    for (uint32_t it = 0;; ++it) {
      unsigned int v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f + r) : "memory");
      if (static_cast<int>(v - static_cast<unsigned int>(p.gate_epoch)) >= 0) break;
      if ((it & 63u) == 63u) {
        if (*abort_flag) return false;
        if (p.status != nullptr && *reinterpret_cast<volatile unsigned int*>(p.status) != 0u) return false;
        uint64_t now;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
        if (t0 == 0) t0 = now;
        if (now - t0 > 2000000000ull) return false;   // 2 s
        __nanosleep(64);
      }
    }
  }
  asm volatile("fence.proxy.async;" ::: "memory");
  return true;
}

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

// ---- work distribution -----------------------------------------------------------------------------
// The output is cut into tiles (m group x n block; m groups vary fastest so CTAs that run together
// share B panels in L2) and, with split-K, each tile's k-blocks into split_k equal ranges. A work
// unit is (tile, k range); CTA c takes units c, c+G, ... A k range that is only part of K is written
// as an fp32 partial tile and a second pass adds the partials and applies the epilogue.
struct Segment {
  int tile, ks, kb0, kb1;
  int sk_tile, piece, n_pieces;   // stream-K tail: index in the tail region, which piece, of how many
};
// Pieces that share tile t of the tail region: workers first..last (the ranges are q k-blocks long).
__host__ __device__ __forceinline__ void sk_tile_pieces(int t, int num_kb, int q, int sk_total, int& first, int& last) {
  first = (t * num_kb) / q;
  const int end = (t + 1) * num_kb < sk_total ? (t + 1) * num_kb : sk_total;
  last = (end - 1) / q;
}
// Units come in two phases. First whole tiles (with split-K: (tile, k range) pairs) dealt round-robin:
// worker w takes units w, w+W, ... Then, when the tile count is not a multiple of W, the k-blocks of
// the left-over tiles laid end to end and cut into W equal ranges, so that the last wave keeps every
// worker busy; the pieces of a tile cut that way are fp32 partial sums that sk_fixup_kernel adds up.
struct Walk {
  int cur, units, tiles_dp, num_kb, kb_per, step;
  int g, g_end, q, sk_total;
  __device__ __forceinline__ Walk(int w, int W, int tiles_, int num_kb_, int split_k, int tiles_dp_, int q_)
      : cur(w), units((q_ > 0 ? tiles_dp_ : tiles_) * split_k), tiles_dp(q_ > 0 ? tiles_dp_ : tiles_),
        num_kb(num_kb_), kb_per((num_kb_ + split_k - 1) / split_k), step(W), q(q_) {
    sk_total = q_ > 0 ? (tiles_ - tiles_dp_) * num_kb_ : 0;
    g = q_ > 0 ? min(w * q_, sk_total) : 0;
    g_end = q_ > 0 ? min(g + q_, sk_total) : 0;
  }
  __device__ __forceinline__ bool next(Segment& s) {
    if (cur < units) {
      s.tile = cur % tiles_dp;
      s.ks = cur / tiles_dp;
      s.kb0 = min(num_kb, s.ks * kb_per);
      s.kb1 = min(num_kb, s.kb0 + kb_per);
      s.sk_tile = 0;
      s.piece = 0;
      s.n_pieces = 1;
      cur += step;
      return true;
    }
    if (g < g_end) {
      const int t = g / num_kb;
      const int kb0 = g - t * num_kb;
      const int len = min(num_kb - kb0, g_end - g);
      s.tile = tiles_dp + t;
      s.ks = 0;
      s.kb0 = kb0;
      s.kb1 = kb0 + len;
      s.sk_tile = t;
      int first, last;
      sk_tile_pieces(t, num_kb, q, sk_total, first, last);
      s.n_pieces = last - first + 1;
      s.piece = g / q - first;
      g += len;
      return true;
    }
    return false;
  }
};

// CG = 1: one CTA per tile. CG = 2 (MT must be 1): the two CTAs of a cluster share a 256-row tile;
// each stages its own 128 rows of A and BN/2 of the weight rows, the even CTA issues
// tcgen05.mma.cta_group::2 for both, and each CTA drains its own 128 accumulator rows. Per SM that
// halves the weight bytes entering shared memory for the same tensor work.
// WIDE (CTA pairs, plain epilogue): a tile of more than 256 columns, computed as two pair MMAs of BN / 2 columns
// per k step into one accumulator of BN columns. A pair MMA takes half of its weight rows from each CTA, so
// each CTA stages quarter `rank` of both halves, one behind the other, and the accumulator columns come out in
// the order of the weight rows. A separate instantiation: the common kernel's instruction stream is untouched.
template <int MT, int EPI, int CG, bool WIDE>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB0,
                    const __grid_constant__ CUtensorMap tmB1, DevParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem_al = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                                ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_al);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kMaxStages;
  uint64_t* tmem_full = bars + 2 * kMaxStages;
  uint64_t* tmem_empty = bars + 2 * kMaxStages + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kMaxStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint8_t* smem = smem_al + 1024;     // ring slots

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  static_assert(CG == 1 || MT == 1, "CTA pairs cover one M tile per CTA");
  static_assert(!WIDE || (CG == 2 && EPI == 0), "wide tiles: CTA pairs, plain epilogue");
  const uint32_t rank = (CG == 2) ? cluster_ctarank() : 0u;   // position in the CTA pair
  const bool leader = rank == 0;
  const int BN = p.bn;                    // tile width = N of one MMA instruction
  const int STAGES = p.stages;
  const int ACC_BUFS = p.acc_bufs;
  const int ACC_COLS = MT * BN;
  const int B_BYTES = (BN / CG) * BK * 2; // weight rows this CTA stages per k-block
  // A CTA that gives up tells its peer too, so the pair unwinds together.
  auto raise_abort = [&]() {
    *abort_flag = 1;
    if (CG == 2)
      st_shared_cluster_u32(mapa_shared(smem_u32(const_cast<int*>(abort_flag)), rank ^ 1u), 1u);
  };
  const int STAGE_BYTES = MT * A_TILE_BYTES + B_BYTES;
  constexpr int A_BYTES = MT * A_TILE_BYTES;
  // Output tile width: the SwiGLU epilogue folds a gate half and an up half of BN/2 columns each.
  const int OUT_BN = (EPI == 1) ? BN / 2 : BN;
  const int m_tiles = (p.M + BM - 1) / BM;
  const int m_groups = (m_tiles + MT * CG - 1) / (MT * CG);
  const int n_blocks = (p.N + OUT_BN - 1) / OUT_BN;
  const int num_kb = (p.K + BK - 1) / BK;
  const int tiles = m_groups * n_blocks;
  const int sk = p.split_k;
  const int worker = blockIdx.x / CG, workers = gridDim.x / CG;   // a CTA, or a CTA pair

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 4 * CG);   // the epilogue warps of every CTA that shares the tile
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB0);
    if (EPI == 1) tma_prefetch_desc(&tmB1);
  }
  if (warp == 1) {
    if (CG == 2) {
      tmem_alloc_pair(tmem_slot, static_cast<uint32_t>(p.tmem_cols));
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, static_cast<uint32_t>(p.tmem_cols));
      tmem_relinquish();
    }
  }
  tc_fence_before();
  if (CG == 2) cluster_sync_all();   // the peer's barriers exist before anything signals them
  else __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0 && lane == 0) {
    // ---------------- TMA producer ----------------
    // ring position kept as (slot, phase) counters: the stage count is a runtime value and a
    // division per k-block would sit on this thread's issue path
    uint32_t it = 0, ph = 0;
    int s = 0;
    bool ok = true;
    Walk walk(worker, workers, tiles, num_kb, sk, p.sk_tiles_dp, p.sk_q);
    Segment sg;
    int gate_seen = -1;     // M tiles up to this one have been seen complete (tiles are walked in row order)
    while (ok && walk.next(sg)) {
      int m_grp, n_blk;
      tile_coords(p, sg.tile, m_groups, n_blocks, m_grp, n_blk);
      const int mt_valid = min(MT, m_tiles - m_grp * MT);
      if (p.gate_flags != nullptr) {
        // last 128-row block of A that this CTA loads for the tile
        const int need = (CG == 2) ? min(m_tiles - 1, m_grp * 2 + static_cast<int>(rank)) : m_grp * MT + mt_valid - 1;
        const int first = (CG == 2) ? need : m_grp * MT;
        for (int mt_i = max(first, gate_seen + 1); mt_i <= need && ok; ++mt_i) {
          if (!wait_gate(p, mt_i, abort_flag)) {
            report_status(p.status, NF_ST_TIMEOUT_PEER_FLAG);
            raise_abort();
            ok = false;
          }
        }
        if (!ok) break;
        if (need > gate_seen) gate_seen = need;
      }
      for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++it, s = (s + 1 == STAGES) ? 0 : s + 1, ph ^= (s == 0)) {
        if (!wait_or_abort(&empty_bar[s], ph ^ 1, abort_flag)) {
          report_status(p.status, NF_ST_TIMEOUT_SMEM_EMPTY);
          raise_abort();
          ok = false;
          break;
        }
        uint8_t* sa = smem + s * STAGE_BYTES;
        uint8_t* sb = sa + A_BYTES;
        if (CG == 2) {
          // Both CTAs' bytes are counted on the even CTA's barrier, which its MMA thread waits on.
          // A tile past the last row or column is still copied in full (zero filled).
          const uint32_t fb = mapa_shared(smem_u32(&full_bar[s]), 0);
          if (leader) mbar_expect_tx(&full_bar[s], 2 * (A_TILE_BYTES + B_BYTES));
          if (EPI == 1)
            tma_load_2d_pair(sb, rank == 0 ? &tmB0 : &tmB1, fb, kb * BK, n_blk * OUT_BN);
          else if (WIDE) {
            const int qrows = BN / 4;
            tma_load_2d_pair(sb, &tmB0, fb, kb * BK, n_blk * BN + static_cast<int>(rank) * qrows);
            tma_load_2d_pair(sb + qrows * (BK * 2), &tmB0, fb, kb * BK,
                             n_blk * BN + BN / 2 + static_cast<int>(rank) * qrows);
          } else
            tma_load_2d_pair(sb, &tmB0, fb, kb * BK, n_blk * BN + static_cast<int>(rank) * (BN / 2));
          tma_load_2d_pair(sa, &tmA, fb, kb * BK, (m_grp * 2 + static_cast<int>(rank)) * BM);
          continue;
        }
        mbar_expect_tx(&full_bar[s], mt_valid * A_TILE_BYTES + B_BYTES);
        if (EPI == 1) {
          tma_load_2d(sb, &tmB0, &full_bar[s], kb * BK, n_blk * OUT_BN);
          tma_load_2d(sb + B_BYTES / 2, &tmB1, &full_bar[s], kb * BK, n_blk * OUT_BN);
        } else {
          tma_load_2d(sb, &tmB0, &full_bar[s], kb * BK, n_blk * BN);
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
          if (mt < mt_valid)
            tma_load_2d(sa + mt * A_TILE_BYTES, &tmA, &full_bar[s], kb * BK, (m_grp * MT + mt) * BM);
      }
    }
    if (CG == 2 && ok) {
      // Every arrival that the even CTA's commits send to this CTA's slot barriers has landed once
      // each slot reads as free again.
      for (int j = 0; j < STAGES; ++j, s = (s + 1 == STAGES) ? 0 : s + 1, ph ^= (s == 0))
        if (!wait_or_abort(&empty_bar[s], ph ^ 1, abort_flag)) break;
    }
    if (!ok && leader) {
      // Drain: give loads already in flight a bounded chance to land before the CTA exits (a
      // pair's loads are all counted on the even CTA's barriers).
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
  } else if (warp == 1 && lane == 0 && leader) {
    // ---------------- MMA issuer (the even CTA of a pair issues for both) ----------------
    const uint32_t idesc = umma_idesc_bf16(BM * CG, WIDE ? BN / 2 : BN);
    uint32_t tcount = 0, ph = 0;
    int s = 0;
    bool ok = true;
    Walk walk(worker, workers, tiles, num_kb, sk, p.sk_tiles_dp, p.sk_q);
    Segment sg;
    while (ok && walk.next(sg)) {
      int m_grp, n_blk_unused;
      tile_coords(p, sg.tile, m_groups, n_blocks, m_grp, n_blk_unused);
      const int mt_valid = (CG == 2) ? 1 : min(MT, m_tiles - m_grp * MT);
      const uint32_t acc = (ACC_BUFS == 2) ? (tcount & 1) : 0;
      const uint32_t acc_ph = (ACC_BUFS == 2) ? ((tcount >> 1) & 1) : (tcount & 1);
      if (!wait_or_abort(&tmem_empty[acc], acc_ph ^ 1, abort_flag)) {
        report_status(p.status, NF_ST_TIMEOUT_TMEM_EMPTY);
        raise_abort();
        break;
      }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * ACC_COLS;
      for (int kb = sg.kb0; kb < sg.kb1; ++kb, s = (s + 1 == STAGES) ? 0 : s + 1, ph ^= (s == 0)) {
        if (!wait_or_abort(&full_bar[s], ph, abort_flag)) {
          report_status(p.status, NF_ST_TIMEOUT_SMEM_FULL);
          raise_abort();
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES);
        const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          if (mt < mt_valid) {
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              const uint64_t da = umma_desc_k_sw128(a_addr + mt * A_TILE_BYTES + k * UMMA_K * 2);
              const uint64_t db = umma_desc_k_sw128(b_addr + k * UMMA_K * 2);
              if (CG == 2) umma_bf16_ss_pair(d_tmem, da, db, idesc, (kb != sg.kb0 || k != 0) ? 1u : 0u);
              else umma_bf16_ss(d_tmem + mt * BN, da, db, idesc, (kb != sg.kb0 || k != 0) ? 1u : 0u);
              if (WIDE)   // second half of the tile: the weight rows staged behind the first quarter
                umma_bf16_ss_pair(d_tmem + BN / 2, da,
                                  umma_desc_k_sw128(b_addr + (BN / 4) * (BK * 2) + k * UMMA_K * 2), idesc,
                                  (kb != sg.kb0 || k != 0) ? 1u : 0u);
            }
          }
        }
        // the stage is free (in both CTAs of a pair) once these MMAs have read it
        if (CG == 2) {
          umma_commit_pair_both(&empty_bar[s]);
        } else {
          umma_commit(&empty_bar[s]);
        }
      }
      if (ok) {
        if (CG == 2) {
          umma_commit_pair_both(&tmem_full[acc]);
        } else {
          umma_commit(&tmem_full[acc]);
        }
      }
      ++tcount;
    }
  } else if (warp >= 2) {
    // ---------------- epilogue (4 warps, 128 threads) ----------------
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    uint32_t tcount = 0;
    Walk walk(worker, workers, tiles, num_kb, sk, p.sk_tiles_dp, p.sk_q);
    Segment sg;
    while (walk.next(sg)) {
      int m_grp, n_blk;
      tile_coords(p, sg.tile, m_groups, n_blocks, m_grp, n_blk);
      const int m_first = (m_grp * CG + static_cast<int>(rank)) * MT;   // first M tile this CTA drains
      const int mt_valid = min(MT, m_tiles - m_first);                  // <= 0: tile past the last row
      const uint32_t acc = (ACC_BUFS == 2) ? (tcount & 1) : 0;
      const uint32_t acc_ph = (ACC_BUFS == 2) ? ((tcount >> 1) & 1) : (tcount & 1);
      ++tcount;
      if (!wait_or_abort(&tmem_full[acc], acc_ph, abort_flag)) {
        if (lane == 0) report_status(p.status, NF_ST_TIMEOUT_TMEM_FULL);
        raise_abort();
        break;
      }
      __syncwarp();
      tc_fence_after();
      const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * ACC_COLS;
      // a k range that received no k-blocks contributes zeros (its accumulator was never written)
      const bool empty_range = sg.kb0 >= sg.kb1;
      // Stream-K tail: the fp32 partial copies of this tile (one slot per piece and CTA of a pair).
      const long long slot_floats = static_cast<long long>(MT) * BM * BN;
      float* const sk_tile_base = (EPI != 2 && sg.n_pieces > 1)
          ? p.sk_partial + (static_cast<long long>(sg.sk_tile) * p.sk_max_pieces * CG) * slot_floats
          : nullptr;
      // mode 0: epilogue to the output; mode 1: raw accumulators to this piece's slot.
      auto drain = [&](const int mode) {
#pragma unroll 1
        for (int mt = 0; mt < mt_valid; ++mt) {
          const int row = (m_first + mt) * BM + q * 32 + lane;
          const bool row_ok = row < p.M;
          const long long row_local = static_cast<long long>(mt * BM + q * 32 + lane) * BN;
          __nv_bfloat16* drow = p.D + static_cast<long long>(row) * p.ldd;
          const __nv_bfloat16* crow =
              (EPI == 0 && p.C != nullptr) ? p.C + static_cast<long long>(row) * p.ldc : nullptr;
          const int tile_col_end = min(p.N, (n_blk + 1) * OUT_BN);   // columns past it belong to the next tile
#pragma unroll 1
          for (int c = 0; c * 32 < OUT_BN; ++c) {
            uint32_t r[32];
            float v[32];
            const bool tail16 = (c * 32 + 16 == OUT_BN);               // width = 32k + 16: last chunk is half
            const int nval = tail16 ? 16 : 32;
            if (tail16) tmem_ld_32x32b_x16(t_lane + mt * BN + c * 32, r);
            else tmem_ld_32x32b_x32(t_lane + mt * BN + c * 32, r);
            if (EPI == 1) {
              uint32_t uu[32];
              if (tail16) tmem_ld_32x32b_x16(t_lane + mt * BN + BN / 2 + c * 32, uu);
              else tmem_ld_32x32b_x32(t_lane + mt * BN + BN / 2 + c * 32, uu);
              tmem_ld_wait();
              float gsum[32], usum[32];
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                gsum[j] = __uint_as_float(r[j]);
                usum[j] = __uint_as_float(uu[j]);
              }
              if (mode == 1) {
                if (row_ok) {
                  float* own = sk_tile_base + (static_cast<long long>(sg.piece) * CG + rank) * slot_floats + row_local;
#pragma unroll
                  for (int g4 = 0; g4 < 8; ++g4)
                    if (g4 * 4 < nval) {
                      __stcg(reinterpret_cast<float4*>(own + c * 32) + g4,
                             make_float4(gsum[g4 * 4], gsum[g4 * 4 + 1], gsum[g4 * 4 + 2], gsum[g4 * 4 + 3]));
                      __stcg(reinterpret_cast<float4*>(own + BN / 2 + c * 32) + g4,
                             make_float4(usum[g4 * 4], usum[g4 * 4 + 1], usum[g4 * 4 + 2], usum[g4 * 4 + 3]));
                    }
                }
                continue;
              }
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = gsum[j] / (1.0f + __expf(-gsum[j])) * usum[j];
            } else {
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = empty_range ? 0.f : __uint_as_float(r[j]);
              if (EPI == 0 && mode == 1) {
                if (row_ok) {
                  float* own = sk_tile_base + (static_cast<long long>(sg.piece) * CG + rank) * slot_floats + row_local;
#pragma unroll
                  for (int g4 = 0; g4 < 8; ++g4)
                    if (g4 * 4 < nval)
                      __stcg(reinterpret_cast<float4*>(own + c * 32) + g4,
                             make_float4(v[g4 * 4], v[g4 * 4 + 1], v[g4 * 4 + 2], v[g4 * 4 + 3]));
                }
                continue;
              }
            }
            const int col0 = n_blk * OUT_BN + c * 32;
            if (EPI == 0 && p.partial != nullptr) {
              if (row_ok && col0 < tile_col_end) {
                float* prow = p.partial + (static_cast<long long>(sg.ks) * p.M + row) * p.N;
#pragma unroll
                for (int g4 = 0; g4 < 8; ++g4) {
                  const int col = col0 + g4 * 4;
                  if (col < tile_col_end)
                    *reinterpret_cast<float4*>(prow + col) =
                        make_float4(v[g4 * 4], v[g4 * 4 + 1], v[g4 * 4 + 2], v[g4 * 4 + 3]);
                }
              }
              continue;
            }
            if (EPI == 2 && p.rs_staged) {
              // Staged push: this lane's 32 columns go to its row of the warp's staging piece; when a
              // run of 128 columns (or the tile's last columns) is complete, one bulk copy per lane
              // sends the row's run to the owner's slab. A lane only ever reads back what it wrote, so
              // the generic -> async proxy fence is all the ordering the copy needs.
              uint8_t* stage_row = smem + STAGES * STAGE_BYTES + (q * 32 + lane) * kRsRowPitch;
              // the bulk copy of the previous run reads this row: it must be done reading before the first
              // write of a new run (waiting here, not right after the copy, lets the copy run under the
              // accumulator loads in between)
              if ((c & 3) == 0) tma_store_wait_read<0>();
#pragma unroll
              for (int g8 = 0; g8 < 4; ++g8) {
                if (g8 * 8 < nval) {
                  const float* vv = v + g8 * 8;
                  uint4 o;
                  o.x = pack_bf16x2(vv[0], vv[1]);
                  o.y = pack_bf16x2(vv[2], vv[3]);
                  o.z = pack_bf16x2(vv[4], vv[5]);
                  o.w = pack_bf16x2(vv[6], vv[7]);
                  *reinterpret_cast<uint4*>(stage_row + (c & 3) * 64 + g8 * 16) = o;
                }
              }
              const bool run_done = (c & 3) == 3 || (c + 1) * 32 >= OUT_BN;
              if (run_done) {
                const int run_col0 = n_blk * OUT_BN + (c & ~3) * 32;
                int run_end = n_blk * OUT_BN + c * 32 + nval;
                if (run_end > tile_col_end) run_end = tile_col_end;
                fence_proxy_async_smem();
                if (row_ok && run_end > run_col0) {
                  const int owner = row % p.rs_nranks;
                  __nv_bfloat16* srow = reinterpret_cast<__nv_bfloat16*>(p.rs_heap[owner] + p.rs_slab_off) +
                                        (static_cast<long long>(p.rs_rank) * p.rs_rows_cap + row / p.rs_nranks) * p.N;
                  bulk_store_1d(srow + run_col0, stage_row, static_cast<uint32_t>(run_end - run_col0) * 2u);
                }
                tma_store_commit();
              }
              continue;
            }
            if (EPI == 2) {
              // push the partial row to its owner's slab (posted NVLink stores; the flag raised at
              // the end of the kernel orders them for the reader)
              if (row_ok && col0 < tile_col_end) {
                const int owner = row % p.rs_nranks;
                __nv_bfloat16* srow = reinterpret_cast<__nv_bfloat16*>(p.rs_heap[owner] + p.rs_slab_off) +
                                      (static_cast<long long>(p.rs_rank) * p.rs_rows_cap + row / p.rs_nranks) * p.N;
#pragma unroll
                for (int g8 = 0; g8 < 4; ++g8) {
                  const int col = col0 + g8 * 8;
                  if (col < tile_col_end) {
                    const float* vv = v + g8 * 8;
                    uint4 o;
                    o.x = pack_bf16x2(vv[0], vv[1]);
                    o.y = pack_bf16x2(vv[2], vv[3]);
                    o.z = pack_bf16x2(vv[4], vv[5]);
                    o.w = pack_bf16x2(vv[6], vv[7]);
                    *reinterpret_cast<uint4*>(srow + col) = o;
                  }
                }
              }
              continue;
            }
            if (row_ok && col0 < tile_col_end) {
#pragma unroll
              for (int g8 = 0; g8 < 4; ++g8) {
                const int col = col0 + g8 * 8;
                if (col < tile_col_end) {  // N is a multiple of 8
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
        }
      };
      // A piece of a tile that several workers share leaves its partial sums in its slot; a second
      // kernel adds the pieces up and applies the epilogue.
      if (sk_tile_base != nullptr) drain(1);
      else drain(0);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (CG == 2) mbar_arrive_cluster(mapa_shared(smem_u32(&tmem_empty[acc]), 0));
        else mbar_arrive(&tmem_empty[acc]);
      }
    }
  }

  if (EPI == 2) {
    tma_store_wait<0>();                    // bulk copies of the staged form have been written
    __threadfence_system();                 // this thread's pushes are ordered before the flag below
  }
  tc_fence_before();
  // Nothing of the pair may still signal this CTA's barriers or read its shared memory or TMEM once
  // it has exited, so the pair leaves together.
  __syncwarp();
  if (CG == 2) cluster_sync_all();
  else __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    if (CG == 2) tmem_dealloc_pair(tmem_base, static_cast<uint32_t>(p.tmem_cols));
    else tmem_dealloc(tmem_base, static_cast<uint32_t>(p.tmem_cols));
  }
  if (EPI == 2 && threadIdx.x == 0) {
    // The last CTA to get here tells every rank that this rank's partial rows have been pushed.
    // Flag block layout (collectives.cu): ready[8], done[8], cta_counter.
    unsigned int* mine = reinterpret_cast<unsigned int*>(p.rs_heap[p.rs_rank] + p.rs_flag_off);
    const unsigned int prev = atomicAdd(mine + 16, 1u);
    if (prev == gridDim.x - 1) {
      mine[16] = 0;
      __threadfence_system();
      for (int r = 0; r < p.rs_nranks; ++r) {
        unsigned int* flag = reinterpret_cast<unsigned int*>(p.rs_heap[r] + p.rs_flag_off) + p.rs_rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(static_cast<unsigned int>(p.rs_epoch))
                     : "memory");
      }
    }
  }
}

// Reduce-scatter epilogue with nothing to push (an empty nano-batch): the consumer still waits for
// this rank's ready flag, so raise it.
__global__ void rs_signal_only_kernel(DevParams p) {
  if (threadIdx.x < p.rs_nranks) {
    unsigned int* flag = reinterpret_cast<unsigned int*>(p.rs_heap[threadIdx.x] + p.rs_flag_off) + p.rs_rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(static_cast<unsigned int>(p.rs_epoch))
                 : "memory");
  }
}

inline int sm_count() { return device_sm_count(); }

// Split-K second pass: D = sum_s partial[s] (+ bias) (+ beta * C), fp32 -> bf16.
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(DevParams p) {
  const long long total = static_cast<long long>(p.M) * (p.N >> 3);
  const long long slab = static_cast<long long>(p.M) * p.N;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < total; i += 256ll * gridDim.x) {
    const int row = static_cast<int>(i / (p.N >> 3));
    const int col = static_cast<int>(i % (p.N >> 3)) * 8;
    float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int s = 0; s < p.split_k; ++s) {
      const float4* src = reinterpret_cast<const float4*>(p.partial + s * slab + static_cast<long long>(row) * p.N + col);
      const float4 a = src[0], b = src[1];
      v[0] += a.x; v[1] += a.y; v[2] += a.z; v[3] += a.w;
      v[4] += b.x; v[5] += b.y; v[6] += b.z; v[7] += b.w;
    }
    if (p.bias != nullptr) {
      const uint4 bv = *reinterpret_cast<const uint4*>(p.bias + col);
      const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(bw[j]);
        v[2 * j] += f.x;
        v[2 * j + 1] += f.y;
      }
    }
    if (p.C != nullptr) {
      const uint4 cv = *reinterpret_cast<const uint4*>(p.C + static_cast<long long>(row) * p.ldc + col);
      const uint32_t cw[4] = {cv.x, cv.y, cv.z, cv.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(cw[j]);
        v[2 * j] += p.beta * f.x;
        v[2 * j + 1] += p.beta * f.y;
      }
    }
    uint4 o;
    o.x = pack_bf16x2(v[0], v[1]);
    o.y = pack_bf16x2(v[2], v[3]);
    o.z = pack_bf16x2(v[4], v[5]);
    o.w = pack_bf16x2(v[6], v[7]);
    *reinterpret_cast<uint4*>(p.D + static_cast<long long>(row) * p.ldd + col) = o;
  }
}

// Split-K second pass with the RMSNorm of the result folded in: one CTA per row (N <= 16384), every
// thread keeps its columns of the row in registers, so the norm costs one block reduction and one
// more store instead of a kernel that reads the row back.
constexpr int kRowVec = 8;   // 8-column groups per thread: 8 * 8 * 256 threads = 16384 columns
__global__ void __launch_bounds__(256)
splitk_reduce_norm_kernel(DevParams p) {
  __shared__ float red[8];
  const int nvec = p.N >> 3;
  const long long slab = static_cast<long long>(p.M) * p.N;
  for (int row = blockIdx.x; row < p.M; row += gridDim.x) {
    float v[kRowVec][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kRowVec; ++i) {
      const int vi = threadIdx.x + i * 256;
      if (vi < nvec) {
        const int col = vi * 8;
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] = 0.f;
        for (int sidx = 0; sidx < p.split_k; ++sidx) {
          const float4* src = reinterpret_cast<const float4*>(p.partial + sidx * slab + static_cast<long long>(row) * p.N + col);
          const float4 a = src[0], b = src[1];
          v[i][0] += a.x; v[i][1] += a.y; v[i][2] += a.z; v[i][3] += a.w;
          v[i][4] += b.x; v[i][5] += b.y; v[i][6] += b.z; v[i][7] += b.w;
        }
        if (p.bias != nullptr) {
          const uint4 bv = *reinterpret_cast<const uint4*>(p.bias + col);
          const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = unpack_bf16x2(bw[j]);
            v[i][2 * j] += f.x;
            v[i][2 * j + 1] += f.y;
          }
        }
        if (p.C != nullptr) {
          const uint4 cv = *reinterpret_cast<const uint4*>(p.C + static_cast<long long>(row) * p.ldc + col);
          const uint32_t cw[4] = {cv.x, cv.y, cv.z, cv.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = unpack_bf16x2(cw[j]);
            v[i][2 * j] += p.beta * f.x;
            v[i][2 * j + 1] += p.beta * f.y;
          }
        }
        uint4 o;
        o.x = pack_bf16x2(v[i][0], v[i][1]);
        o.y = pack_bf16x2(v[i][2], v[i][3]);
        o.z = pack_bf16x2(v[i][4], v[i][5]);
        o.w = pack_bf16x2(v[i][6], v[i][7]);
        *reinterpret_cast<uint4*>(p.D + static_cast<long long>(row) * p.ldd + col) = o;
        // normalise what was stored (bf16-rounded), as the standalone norm kernel would read it
        const uint32_t ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16x2(ow[j]);
          v[i][2 * j] = f.x;
          v[i][2 * j + 1] = f.y;
          ss += f.x * f.x + f.y * f.y;
        }
      }
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = (threadIdx.x & 31) < 8 ? red[threadIdx.x & 31] : 0.f;
    tot = warp_sum(tot);
    __syncthreads();
    const float inv = rsqrtf(tot / static_cast<float>(p.N) + p.norm_eps);
#pragma unroll
    for (int i = 0; i < kRowVec; ++i) {
      const int vi = threadIdx.x + i * 256;
      if (vi < nvec) {
        const uint4 ww = *reinterpret_cast<const uint4*>(p.norm_w + vi * 8);
        const uint32_t wv[4] = {ww.x, ww.y, ww.z, ww.w};
        uint32_t ov[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 g = unpack_bf16x2(wv[j]);
          ov[j] = pack_bf16x2(v[i][2 * j] * inv * g.x, v[i][2 * j + 1] * inv * g.y);
        }
        *reinterpret_cast<uint4*>(p.norm_out + static_cast<long long>(row) * p.norm_ld + vi * 8) =
            make_uint4(ov[0], ov[1], ov[2], ov[3]);
      }
    }
  }
}

// Stream-K tail, second pass: for every tile of the tail region that was cut into pieces, add the
// pieces' fp32 partial sums and apply the epilogue. One thread per 8 output columns of a row; the
// loads of the pieces are independent, so many are in flight per thread.
struct FixupGeom {
  int mt, cg, bn, out_bn, m_groups, num_kb, rest;
};
template <int EPI>
__global__ void __launch_bounds__(256)
sk_fixup_kernel(DevParams p, FixupGeom f) {
  const int rows_cta = f.mt * BM;
  const int groups = f.out_bn / 8;
  const long long slot_floats = static_cast<long long>(rows_cta) * f.bn;
  const int sk_total = f.rest * f.num_kb;
  const long long per_cta = static_cast<long long>(rows_cta) * groups;
  const long long per_tile = per_cta * f.cg;
  const long long total = per_tile * f.rest;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < total; i += 256ll * gridDim.x) {
    const int t = static_cast<int>(i / per_tile);
    long long r = i - t * per_tile;
    const int rank = static_cast<int>(r / per_cta);
    r -= rank * per_cta;
    const int row_local = static_cast<int>(r / groups);
    const int gcol = static_cast<int>(r - static_cast<long long>(row_local) * groups) * 8;
    int first, last;
    sk_tile_pieces(t, f.num_kb, p.sk_q, sk_total, first, last);
    const int n_pieces = last - first + 1;
    if (n_pieces < 2) continue;   // written whole by its only piece
    const int tile = p.sk_tiles_dp + t;
    const int m_grp = tile % f.m_groups, n_blk = tile / f.m_groups;
    const int row = (m_grp * f.cg + rank) * rows_cta + row_local;
    const int col = n_blk * f.out_bn + gcol;
    if (row >= p.M || col >= p.N) continue;
    const float* base = p.sk_partial + (static_cast<long long>(t) * p.sk_max_pieces * f.cg + rank) * slot_floats +
                        static_cast<long long>(row_local) * f.bn + gcol;
    float a[8] = {0, 0, 0, 0, 0, 0, 0, 0}, u[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll 4
    for (int pi = 0; pi < n_pieces; ++pi) {
      const float* src = base + static_cast<long long>(pi) * f.cg * slot_floats;
      const float4 x0 = __ldcg(reinterpret_cast<const float4*>(src));
      const float4 x1 = __ldcg(reinterpret_cast<const float4*>(src) + 1);
      a[0] += x0.x; a[1] += x0.y; a[2] += x0.z; a[3] += x0.w;
      a[4] += x1.x; a[5] += x1.y; a[6] += x1.z; a[7] += x1.w;
      if (EPI == 1) {
        const float4 y0 = __ldcg(reinterpret_cast<const float4*>(src + f.bn / 2));
        const float4 y1 = __ldcg(reinterpret_cast<const float4*>(src + f.bn / 2) + 1);
        u[0] += y0.x; u[1] += y0.y; u[2] += y0.z; u[3] += y0.w;
        u[4] += y1.x; u[5] += y1.y; u[6] += y1.z; u[7] += y1.w;
      }
    }
    if (EPI == 1) {
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] = a[j] / (1.0f + __expf(-a[j])) * u[j];
    } else {
      if (p.bias != nullptr) {
        const uint4 bv = *reinterpret_cast<const uint4*>(p.bias + col);
        const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 fl = unpack_bf16x2(bw[j]);
          a[2 * j] += fl.x;
          a[2 * j + 1] += fl.y;
        }
      }
      if (p.C != nullptr) {
        const uint4 cv = *reinterpret_cast<const uint4*>(p.C + static_cast<long long>(row) * p.ldc + col);
        const uint32_t cw[4] = {cv.x, cv.y, cv.z, cv.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 fl = unpack_bf16x2(cw[j]);
          a[2 * j] += p.beta * fl.x;
          a[2 * j + 1] += p.beta * fl.y;
        }
      }
    }
    uint4 o;
    o.x = pack_bf16x2(a[0], a[1]);
    o.y = pack_bf16x2(a[2], a[3]);
    o.z = pack_bf16x2(a[4], a[5]);
    o.w = pack_bf16x2(a[6], a[7]);
    *reinterpret_cast<uint4*>(p.D + static_cast<long long>(row) * p.ldd + col) = o;
  }
}

constexpr int kSmemMax = 227 * 1024;

// Stream-K tail: with `tiles` tiles on `workers` workers, the tiles_dp tiles of the full waves are
// whole-tile units; the k-blocks of the rest are cut into ranges of q (>= 8, so a piece is worth its
// set-up), one per worker.
struct SkPlan {
  int tiles_dp, q, max_pieces, rest;
};
inline SkPlan plan_stream_k(int tiles, int workers, int num_kb) {
  SkPlan pl{tiles, 0, 0, 0};
  const int rest = tiles % workers;
  if (rest == 0 || num_kb < 2) return pl;
  int q = (static_cast<long long>(rest) * num_kb + workers - 1) / workers;
  const int q_min = num_kb < 8 ? num_kb : 8;
  if (q < q_min) q = q_min;
  if (q >= num_kb) return pl;           // nothing would be cut
  pl.tiles_dp = tiles - rest;
  pl.q = q;
  pl.max_pieces = (num_kb + q - 1) / q + 1;
  pl.rest = rest;
  return pl;
}

template <int MT, int EPI, int CG, bool WIDE>
int launch_impl(const nfk_gemm_params& g, int bn, int split_k, bool stream_k, cudaStream_t stream) {
  int budget = g.smem_budget_kb > 0 ? g.smem_budget_kb * 1024 : kSmemMax;
  if (budget > kSmemMax) budget = kSmemMax;
  const bool rs_staged = EPI == 2 && g.rs_staged != 0;
  const Geom geo = make_geom(bn, MT, EPI == 1, budget, CG, rs_staged ? kRsStageBytes : 0);
  if (geo.stages < 2) return NF_ERR_BAD_ARG;      // shared-memory budget too small for this tile
  CUtensorMap tmA, tmB0, tmB1;
  int rc = make_tmap_bf16_2d(&tmA, g.A, g.M, g.K, g.lda, BM, BK);
  if (rc != NF_OK) return rc;
  // rows of B that one TMA copy brings in: a whole tile, a SwiGLU half, or a CTA pair's half
  // (wide tiles: a quarter of the tile per copy, two copies per CTA)
  const int b_box = (EPI == 1) ? geo.out_bn : (WIDE ? bn / 4 : bn / CG);
  rc = make_tmap_bf16_2d(&tmB0, g.B, g.N, g.K, g.ldb, b_box, BK);
  if (rc != NF_OK) return rc;
  if (EPI == 1) {
    rc = make_tmap_bf16_2d(&tmB1, g.B2, g.N, g.K, g.ldb, b_box, BK);
    if (rc != NF_OK) return rc;
  } else {
    tmB1 = tmB0;
  }
  // function attributes and occupancy are per device: one slot per device this process drives
  static bool attr_set_dev[kMaxDevices] = {false};
  static int max_workers_dev[kMaxDevices] = {0};    // CTAs (or CTA pairs) that can be resident at once
  bool& attr_set = attr_set_dev[device_slot()];
  int& max_workers = max_workers_dev[device_slot()];
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_tcgen05_kernel<MT, EPI, CG, WIDE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kSmemMax) != cudaSuccess)
      return NF_ERR_CUDA;
    // Always the largest shared-memory split: with a reduced budget (smem_budget_kb) the SM then
    // keeps room for the CTAs of a kernel that runs beside this one, whichever of the two came first.
    (void)cudaFuncSetAttribute(gemm_tcgen05_kernel<MT, EPI, CG, WIDE>, cudaFuncAttributePreferredSharedMemoryCarveout,
                               cudaSharedmemCarveoutMaxShared);
    (void)cudaGetLastError();
    max_workers = sm_count() / CG;
    if (CG == 2) {
      // Pairs must sit on two SMs of one GPC; ask how many fit so that no pair waits for a second wave.
      cudaLaunchConfig_t qc = {};
      qc.gridDim = dim3(sm_count() / 2 * 2);
      qc.blockDim = dim3(kGemmThreads);
      qc.dynamicSmemBytes = kSmemMax;
      cudaLaunchAttribute qa[1];
      qa[0].id = cudaLaunchAttributeClusterDimension;
      qa[0].val.clusterDim.x = 2;
      qa[0].val.clusterDim.y = 1;
      qa[0].val.clusterDim.z = 1;
      qc.attrs = qa;
      qc.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, gemm_tcgen05_kernel<MT, EPI, CG, WIDE>, &qc) == cudaSuccess && n > 0 &&
          n < max_workers)
        max_workers = n;
      else
        (void)cudaGetLastError();
    }
    attr_set = true;
  }
  const int m_tiles = (g.M + BM - 1) / BM;
  const int m_groups = (m_tiles + MT * CG - 1) / (MT * CG);
  const int n_blocks = (g.N + geo.out_bn - 1) / geo.out_bn;
  const int units = m_groups * n_blocks * split_k;
  int workers = (g.num_ctas > 0 ? g.num_ctas : sm_count()) / CG;
  if (workers > max_workers) workers = max_workers;
  if (workers < 1) workers = 1;
  // stream_k 3: one work unit per CTA (or CTA pair), more CTAs than fit at once; the hardware block
  // scheduler deals the units out as CTAs retire, so an SM that another kernel's CTAs slow down takes
  // fewer of them instead of holding the launch back (no CTA of this kernel waits for another one)
  const bool hw_dealt = g.stream_k == 3 && g.gate_flags == nullptr;
  if (hw_dealt) {
    workers = units;
    stream_k = false;
  }
  SkPlan sk{m_groups * n_blocks, 0, 0, 0};
  if (stream_k && split_k == 1 && EPI != 2 && g.workspace != nullptr) {
    sk = plan_stream_k(m_groups * n_blocks, workers, (g.K + BK - 1) / BK);
    const long long need = static_cast<long long>(sk.rest) * sk.max_pieces * CG * MT * BM * bn * 4;
    if (sk.q > 0 && need > g.workspace_bytes)
      sk = SkPlan{m_groups * n_blocks, 0, 0, 0};
  }
  if (sk.q == 0 && workers > units) workers = units;
  const int ctas = workers * CG;
  DevParams p;
  p.D = reinterpret_cast<__nv_bfloat16*>(g.D);
  p.C = reinterpret_cast<const __nv_bfloat16*>(g.C);
  p.bias = reinterpret_cast<const __nv_bfloat16*>(g.bias);
  p.partial = split_k > 1 ? reinterpret_cast<float*>(g.workspace) : nullptr;
  p.sk_partial = sk.q > 0 ? reinterpret_cast<float*>(g.workspace) : nullptr;
  p.sk_tiles_dp = sk.tiles_dp;
  p.sk_q = sk.q;
  p.sk_max_pieces = sk.max_pieces;
  p.ldd = g.ldd;
  p.ldc = g.ldc;
  p.beta = g.beta;
  p.M = g.M;
  p.N = g.N;
  p.K = g.K;
  p.split_k = split_k;
  p.status = g.status;
  p.bn = geo.bn;
  p.stages = geo.stages;
  p.acc_bufs = geo.acc_bufs;
  p.tmem_cols = geo.tmem_cols;
  for (int r = 0; r < 8; ++r) p.rs_heap[r] = reinterpret_cast<char*>(g.rs_heap[r]);
  p.rs_rank = g.rs_rank;
  p.rs_nranks = g.rs_nranks;
  p.rs_rows_cap = g.rs_rows_cap;
  p.rs_epoch = g.rs_epoch;
  p.rs_slab_off = g.rs_slab_off;
  p.rs_flag_off = g.rs_flag_off;
  p.rs_staged = rs_staged ? 1 : 0;
  p.gate_flags = g.gate_flags;
  p.gate_epoch = g.gate_epoch;
  p.gate_nranks = g.gate_nranks;
  if (CG == 2) {
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(ctas);
    lc.blockDim = dim3(kGemmThreads);
    lc.dynamicSmemBytes = geo.smem_bytes;
    lc.stream = stream;
    cudaLaunchAttribute la[1];
    la[0].id = cudaLaunchAttributeClusterDimension;
    la[0].val.clusterDim.x = 2;
    la[0].val.clusterDim.y = 1;
    la[0].val.clusterDim.z = 1;
    lc.attrs = la;
    lc.numAttrs = 1;
    if (cudaLaunchKernelEx(&lc, gemm_tcgen05_kernel<MT, EPI, CG, WIDE>, tmA, tmB0, tmB1, p) != cudaSuccess) {
      (void)cudaGetLastError();
      return NF_ERR_CUDA;
    }
  } else {
    gemm_tcgen05_kernel<MT, EPI, CG, WIDE><<<ctas, kGemmThreads, geo.smem_bytes, stream>>>(tmA, tmB0, tmB1, p);
    if (cudaGetLastError() != cudaSuccess) return NF_ERR_CUDA;
  }
  if (sk.q > 0 && EPI != 2) {
    FixupGeom f{MT, CG, bn, geo.out_bn, m_groups, (g.K + BK - 1) / BK, sk.rest};
    const long long total = static_cast<long long>(sk.rest) * CG * MT * BM * (geo.out_bn / 8);
    long long blocks = (total + 255) / 256;
    if (blocks > sm_count() * 8) blocks = sm_count() * 8;
    sk_fixup_kernel<EPI == 1 ? 1 : 0><<<static_cast<int>(blocks), 256, 0, stream>>>(p, f);
    if (cudaGetLastError() != cudaSuccess) return NF_ERR_CUDA;
  }
  p.norm_w = reinterpret_cast<const __nv_bfloat16*>(g.norm_w);
  p.norm_out = reinterpret_cast<__nv_bfloat16*>(g.norm_out);
  p.norm_ld = g.norm_ld;
  p.norm_eps = g.norm_eps;
  const bool want_norm = EPI == 0 && g.norm_w != nullptr;
  if (split_k > 1 && want_norm && g.N <= kRowVec * 8 * 256) {
    const int blocks = g.M < 16 * sm_count() ? g.M : 16 * sm_count();
    splitk_reduce_norm_kernel<<<blocks, 256, 0, stream>>>(p);
    return cudaGetLastError() == cudaSuccess ? NF_OK : NF_ERR_CUDA;
  }
  if (split_k > 1) {
    const long long total = static_cast<long long>(g.M) * (g.N >> 3);
    long long blocks = (total + 255) / 256;
    if (blocks > 4ll * sm_count()) blocks = 4ll * sm_count();
    splitk_reduce_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(p);
    if (cudaGetLastError() != cudaSuccess) return NF_ERR_CUDA;
  }
  if (want_norm) {
    // the result rows are complete in D (contiguous rows required): a plain norm launch follows
    if (g.ldd != g.N || g.norm_ld != g.N) return NF_ERR_UNSUPPORTED;
    return nfk_rmsnorm(g.norm_out, g.D, g.norm_w, g.M, g.N, g.norm_eps, stream);
  }
  return NF_OK;
}

template <int MT, int EPI, int CG>
int launch(const nfk_gemm_params& g, int bn, int split_k, bool stream_k, cudaStream_t stream) {
  if constexpr (CG == 2 && EPI == 0 && MT == 1) {
    if (bn > 256) return launch_impl<MT, EPI, CG, true>(g, bn, split_k, stream_k, stream);
  }
  if (bn > 256) return NF_ERR_UNSUPPORTED;
  return launch_impl<MT, EPI, CG, false>(g, bn, split_k, stream_k, stream);
}

template <int EPI>
int launch_mt(const nfk_gemm_params& g, int bn, int mt, int cg, int split_k, bool stream_k, cudaStream_t stream) {
  if (cg == 2) return mt == 1 ? launch<1, EPI, 2>(g, bn, split_k, stream_k, stream) : NF_ERR_UNSUPPORTED;
  switch (mt) {
    case 1: return launch<1, EPI, 1>(g, bn, split_k, stream_k, stream);
    case 2: return launch<2, EPI, 1>(g, bn, split_k, stream_k, stream);
    case 4: return launch<4, EPI, 1>(g, bn, split_k, stream_k, stream);
    default: return NF_ERR_UNSUPPORTED;
  }
}

// Tile-shape choice when the caller leaves it open: a small cost model over the candidate shapes.
// A unit (tile x k range) costs its k-blocks times the per-k-block time of the tile shape (the
// larger of tensor time and shared-memory fill time) plus a fixed prologue/epilogue; the GEMM costs
// waves x unit cost, plus the reduce pass when K is split. MT > 1 shapes let one CTA cover several
// M tiles with one weight tile (each weight byte enters shared memory once), which wins when M is
// small and the GEMM is bound by streaming the weight.
struct Shape {
  int bn, mt, split_k, cg;
  bool stream_k;
};
Shape choose_shape(const nfk_gemm_params& g, bool swiglu) {
  const int ctas = g.num_ctas > 0 ? g.num_ctas : sm_count();
  const int m_tiles = (g.M + BM - 1) / BM;
  const int num_kb = (g.K + BK - 1) / BK;
  Shape best{256, 1, 1, 1, false}, best_tail{256, 1, 1, 1, true};
  double best_cost = 1e30, best_tail_cost = 1e30;
  const int cg_lo = g.cta_group == 2 ? 2 : 1, cg_hi = g.cta_group == 1 ? 1 : 2;
  for (int cg = cg_lo; cg <= cg_hi; ++cg) {
  for (int mt = 1; mt <= (cg == 2 ? 1 : 4); mt *= 2) {
   for (int bn = swiglu ? 128 : 64; bn <= 256; bn += 32) {
    if (mt * bn > 512) continue;
    if (swiglu && (bn / 2) % 16 != 0) continue;
    // Several M tiles per CTA only pay off when M is small (weight streaming); with many M tiles
    // the single TMEM accumulator set would serialise epilogue and main loop for nothing.
    if (mt > 1 && (m_tiles > 4 || m_tiles <= mt / 2)) continue;
    if (cg == 2 && m_tiles < 2) continue;    // a pair covers two M tiles
    const int out_bn = swiglu ? bn / 2 : bn;
    const int m_groups = (m_tiles + mt * cg - 1) / (mt * cg);
    const int n_blocks = (g.N + out_bn - 1) / out_bn;
    const int tiles = m_groups * n_blocks;
    const int mt_eff = m_tiles < mt ? m_tiles : mt;
    // per k-block and SM: tensor time (us) at ~11 TFLOP/s, shared-memory fill at ~100 GB/s (a CTA
    // of a pair stages only half of the weight tile); measured, a pair's k-block never takes less
    // than ~0.36 us whatever the tile width
    const double t_mma = 2.0 * BM * mt_eff * bn * BK / 11.0e6;
    const double t_fill = (mt_eff * 16384.0 + bn * 128.0 / cg) / 100.0e3;
    double t_kb = t_mma > t_fill ? t_mma : t_fill;
    if (cg == 2 && t_kb < 0.36) t_kb = 0.36;
    const int max_sk = (swiglu || g.workspace == nullptr || g.epilogue == NFK_EPI_REDUCE_SCATTER) ? 1 : 8;
    for (int sk = 1; sk <= max_sk; ++sk) {
      if (sk > 1 && (num_kb / sk < 8 ||
                     static_cast<long long>(sk) * g.M * g.N * 4 > g.workspace_bytes)) break;
      const int units = tiles * sk;
      const int workers = ctas / cg > 0 ? ctas / cg : 1;
      const int waves = (units + workers - 1) / workers;
      const int kb_per = (num_kb + sk - 1) / sk;
      // per unit: prologue + epilogue; the epilogue hides under the next main loop only when TMEM
      // holds two accumulator sets
      const bool single_acc = mt * bn * 2 > 512;
      double cost = waves * (kb_per * t_kb + 2.0 + (single_acc ? 0.012 : 0.003) * mt_eff * bn);
      if (sk > 1) cost += 3.0 + (sk + 1.0) * g.M * static_cast<double>(g.N) * 4.0 / 4.0e6;  // partial write + reduce
      if (cost < best_cost) {
        best_cost = cost;
        best = Shape{bn, mt, sk, cg, false};
      }
      // the same shape with a stream-K tail: full waves as above, then one round of k ranges whose
      // pieces are written out as fp32 and summed by the last piece of each tile
      if (sk == 1 && g.stream_k < 2 && g.workspace != nullptr && g.epilogue != NFK_EPI_REDUCE_SCATTER) {
        const SkPlan pl = plan_stream_k(tiles, workers, num_kb);
        const long long need = static_cast<long long>(pl.rest) * pl.max_pieces * cg * mt * BM * bn * 4;
        if (pl.q > 0 && need <= g.workspace_bytes) {
          const double unit_fixed = 2.0 + (single_acc ? 0.012 : 0.003) * mt_eff * bn;
          const double tile_bytes = mt_eff * BM * bn * 4.0;          // one fp32 copy of a CTA's tile rows
          const double pieces = static_cast<double>(num_kb) / pl.q + 1.0;
          // a worker's range may straddle two tiles; its partial copies leave at ~150 GB/s; the second
          // pass is a launch plus all copies read back at ~3 TB/s
          const double fix_us = 3.0 + pl.rest * cg * pieces * tile_bytes / 3.0e6;
          const double tail = pl.q * t_kb + 2.0 * unit_fixed + tile_bytes / 150.0e3 + fix_us;
          const double c2 = (tiles / workers) * (kb_per * t_kb + unit_fixed) + tail;
          if (c2 < best_tail_cost) {
            best_tail_cost = c2;
            best_tail = Shape{bn, mt, 1, cg, true};
          }
        }
      }
    }
   }
  }
  }
  // The tail's second pass and partial copies are modelled coarsely: take it only for a clear gain.
  if (g.stream_k == 1 && best_tail_cost < 1e30) return best_tail;
  return best_tail_cost < 0.88 * best_cost ? best_tail : best;
}

// Shape of this call: the cost model's, or the caller's pinned one, checked against what is built.
int resolve_shape(const nfk_gemm_params& gp, bool swiglu, bool rs, Shape& s) {
  const nfk_gemm_params* g = &gp;
  s = choose_shape(*g, swiglu);
  if (rs) s.split_k = 1;   // partial tiles go straight to their owners: no K split
  if (g->gate_flags != nullptr) {
    s.split_k = 1;         // gated input: whole tiles in row order only
    s.stream_k = false;
  }
  if (g->tile_n != 0 || g->tile_m != 0) {
    // pinned tile shape: fill in the other dimension with its default, split only on request
    s.bn = g->tile_n != 0 ? g->tile_n : 256;
    s.mt = g->tile_m != 0 ? g->tile_m : 1;
    s.split_k = 1;
    s.cg = g->cta_group == 2 ? 2 : 1;
    s.stream_k = false;
  }
  if (g->stream_k == 1) s.stream_k = true;
  if (g->stream_k >= 2 || s.split_k != 1 || g->gate_flags != nullptr) s.stream_k = false;
  if (s.cg == 2 && s.mt != 1) return NF_ERR_UNSUPPORTED;
  if (g->split_k != 0 && g->gate_flags == nullptr) s.split_k = g->split_k;
  if (s.split_k < 1 || s.split_k > 16) return NF_ERR_BAD_ARG;
  if (s.split_k > 1) {
    if (swiglu || g->workspace == nullptr ||
        static_cast<long long>(s.split_k) * g->M * g->N * 4 > g->workspace_bytes)
      return NF_ERR_BAD_ARG;
  }
  // Wider than one MMA instruction (256 columns): CTA pairs, one M tile, plain epilogue (the WIDE kernel).
  const bool wide_ok = s.bn > 256 && s.bn <= 512 && s.bn % 64 == 0 && s.cg == 2 && s.mt == 1 && !swiglu && !rs;
  if (s.bn < 32 || (s.bn > 256 && !wide_ok) || s.bn % 32 != 0 || (s.mt != 1 && s.mt != 2 && s.mt != 4) || s.mt * s.bn > 512)
    return NF_ERR_UNSUPPORTED;
  if (swiglu && (s.bn / 2) % 16 != 0) return NF_ERR_UNSUPPORTED;
  return NF_OK;
}

}  // namespace
}  // namespace nf

// What nfk_gemm_bf16 would launch for these parameters, without launching: tile shape, number of
// tiles and workers, and the stream-K tail (first tile of the tail region, k-blocks per worker, most
// pieces a tile can be cut into). Needs no GPU (the SM count falls back to 148), so planners and
// tests can check the work distribution on any machine.
extern "C" int nfk_gemm_describe(const nfk_gemm_params* g, nfk_gemm_plan* out) {
  using namespace nf;
  if (g == nullptr || out == nullptr || g->M <= 0 || g->N <= 0 || g->K <= 0) return NF_ERR_BAD_ARG;
  const bool swiglu = g->epilogue == NFK_EPI_SWIGLU, rs = g->epilogue == NFK_EPI_REDUCE_SCATTER;
  Shape s;
  const int rc = resolve_shape(*g, swiglu, rs, s);
  if (rc != NF_OK) return rc;
  int budget = g->smem_budget_kb > 0 ? g->smem_budget_kb * 1024 : kSmemMax;
  if (budget > kSmemMax) budget = kSmemMax;
  const Geom geo = make_geom(s.bn, s.mt, swiglu, budget, s.cg, (rs && g->rs_staged) ? kRsStageBytes : 0);
  if (geo.stages < 2) return NF_ERR_BAD_ARG;
  const int m_tiles = (g->M + BM - 1) / BM;
  const int m_groups = (m_tiles + s.mt * s.cg - 1) / (s.mt * s.cg);
  const int n_blocks = (g->N + geo.out_bn - 1) / geo.out_bn;
  const int tiles = m_groups * n_blocks;
  int workers = (g->num_ctas > 0 ? g->num_ctas : sm_count()) / s.cg;
  if (workers > sm_count() / s.cg) workers = sm_count() / s.cg;
  if (workers < 1) workers = 1;
  SkPlan sk{tiles, 0, 0, 0};
  if (s.stream_k && s.split_k == 1 && !rs && g->workspace != nullptr) {
    sk = plan_stream_k(tiles, workers, (g->K + BK - 1) / BK);
    const long long need = static_cast<long long>(sk.rest) * sk.max_pieces * s.cg * s.mt * BM * s.bn * 4;
    if (sk.q > 0 && need > g->workspace_bytes) sk = SkPlan{tiles, 0, 0, 0};
  }
  if (sk.q == 0 && workers > tiles * s.split_k) workers = tiles * s.split_k;
  out->tile_n = s.bn;
  out->tile_m = s.mt;
  out->cta_group = s.cg;
  out->split_k = s.split_k;
  out->stream_k = sk.q > 0 ? 1 : 0;
  out->tiles = tiles;
  out->workers = workers;
  out->num_kb = (g->K + BK - 1) / BK;
  out->tail_first_tile = sk.tiles_dp;
  out->tail_range_kb = sk.q;
  out->tail_max_pieces = sk.max_pieces;
  out->stages = geo.stages;
  out->smem_bytes = geo.smem_bytes;
  return NF_OK;
}

extern "C" int nfk_gemm_bf16(const nfk_gemm_params* g, cudaStream_t stream) {
  using namespace nf;
  if (g == nullptr) return NF_ERR_BAD_ARG;
  if (g->M == 0 && g->epilogue == NFK_EPI_REDUCE_SCATTER) {
    if (g->rs_nranks < 1 || g->rs_nranks > 8 || g->rs_rank < 0 || g->rs_rank >= g->rs_nranks) return NF_ERR_BAD_ARG;
    DevParams p{};
    for (int r = 0; r < 8; ++r) p.rs_heap[r] = reinterpret_cast<char*>(g->rs_heap[r]);
    p.rs_rank = g->rs_rank;
    p.rs_nranks = g->rs_nranks;
    p.rs_epoch = g->rs_epoch;
    p.rs_flag_off = g->rs_flag_off;
    rs_signal_only_kernel<<<1, 32, 0, stream>>>(p);
    return cudaGetLastError() == cudaSuccess ? NF_OK : NF_ERR_CUDA;
  }
  if (g->M == 0 || g->N == 0) return NF_OK;  // empty nano-batch: nothing to do
  if (g->A == nullptr || g->B == nullptr) return NF_ERR_BAD_ARG;
  if (g->D == nullptr && g->epilogue != NFK_EPI_REDUCE_SCATTER) return NF_ERR_BAD_ARG;
  if (g->M < 0 || g->N < 0 || g->K <= 0) return NF_ERR_BAD_ARG;
  if (g->K % 8 != 0 || g->N % 8 != 0 || g->lda % 8 != 0 || g->ldb % 8 != 0 || g->ldd % 8 != 0)
    return NF_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(g->D) & 15) != 0) return NF_ERR_BAD_ARG;
  if (g->C != nullptr && ((reinterpret_cast<uintptr_t>(g->C) & 15) != 0 || g->ldc % 8 != 0))
    return NF_ERR_BAD_ARG;
  if (g->workspace != nullptr && (reinterpret_cast<uintptr_t>(g->workspace) & 15) != 0) return NF_ERR_BAD_ARG;
  const bool swiglu = g->epilogue == NFK_EPI_SWIGLU;
  if (swiglu && g->B2 == nullptr) return NF_ERR_BAD_ARG;
  const bool rs = g->epilogue == NFK_EPI_REDUCE_SCATTER;
  if (g->gate_flags != nullptr &&
      (rs || g->gate_nranks < 1 || g->gate_nranks > 8 || (reinterpret_cast<uintptr_t>(g->gate_flags) & 3) != 0))
    return NF_ERR_BAD_ARG;
  if (rs) {
    if (g->rs_nranks < 1 || g->rs_nranks > 8 || g->rs_rank < 0 || g->rs_rank >= g->rs_nranks ||
        g->rs_rows_cap * g->rs_nranks < g->M || g->rs_slab_off % 16 != 0 || g->rs_flag_off % 16 != 0 ||
        g->split_k > 1)
      return NF_ERR_BAD_ARG;
    for (int r = 0; r < g->rs_nranks; ++r)
      if (g->rs_heap[r] == nullptr) return NF_ERR_BAD_ARG;
  }

  Shape s;
  const int rcs = resolve_shape(*g, swiglu, rs, s);
  if (rcs != NF_OK) return rcs;
  if (swiglu) {
    if ((s.bn / 2) % 16 != 0) return NF_ERR_UNSUPPORTED;
    return launch_mt<1>(*g, s.bn, s.mt, s.cg, 1, s.stream_k, stream);
  }
  if (rs) return launch_mt<2>(*g, s.bn, s.mt, s.cg, 1, false, stream);
  return launch_mt<0>(*g, s.bn, s.mt, s.cg, s.split_k, s.stream_k, stream);
}
