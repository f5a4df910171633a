// C ABI of libnanoflow_kernels.so. Every entry point takes raw device pointers and a CUDA stream,
// launches asynchronously on that stream, allocates nothing, and returns 0 on success or one of
// the NF_ERR_* codes (common.cuh) when an argument is rejected before any launch.
// bf16 tensors are passed as void*; int tensors are int32 unless noted.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ------------------------------------------------------------------------------------------------
// GEMM (gemm.cu)
// ------------------------------------------------------------------------------------------------
enum { NFK_EPI_LINEAR = 0, NFK_EPI_SWIGLU = 1, NFK_EPI_REDUCE_SCATTER = 2 };

typedef struct nfk_gemm_params {
  const void* A;    // [M,K] bf16, row-major, leading dimension lda
  const void* B;    // [N,K] bf16, row-major (nn.Linear weight layout); gate weight for SwiGLU
  const void* B2;   // SwiGLU only: up weight [N,K]
  void* D;          // [M,N] bf16
  const void* C;    // optional residual [M,N]: D = A*B^T + bias + beta*C
  const void* bias; // optional [N] bf16
  long long lda, ldb, ldd, ldc;
  float beta;
  int M, N, K;
  int epilogue;     // NFK_EPI_*
  int tile_n;       // 0 = choose; tile width in weight rows: a multiple of 32 up to 256
  int num_ctas;     // CTA budget of the persistent grid; 0 = one per SM
  unsigned int* status;  // optional device word: first non-zero NF_ST_* code wins
  int tile_m;       // 0 = choose; number of 128-row M tiles one CTA covers: 1 / 2 / 4
  int split_k;      // 0 = choose; > 1 needs `workspace` (fp32 partials, split_k*M*N*4 bytes)
  void* workspace;  // scratch for fp32 partial sums (split-K, stream-K tail); GEMMs that may overlap need their own
  long long workspace_bytes;
  // NFK_EPI_REDUCE_SCATTER: the epilogue does not write D; it pushes every bf16 partial row straight
  // into the slab of the rank that owns the row (row i belongs to rank i % rs_nranks), over NVLink:
  //   heap[owner] + rs_slab_off + ((rs_rank * rs_rows_cap + i / rs_nranks) * N + col) * 2
  // and, once all CTAs are done, raises ready[rs_rank] = rs_epoch in the flag block at rs_flag_off
  // on every rank. nfk_allreduce with src_mode 1 then reduces the slabs locally.
  void* rs_heap[8];
  int rs_rank, rs_nranks;
  long long rs_slab_off;
  int rs_rows_cap;
  long long rs_flag_off;
  int rs_epoch;
  int smem_budget_kb;  // 0 = all 227 KB; smaller leaves shared memory for a kernel meant to share the SM
  int cta_group;       // 0 = let the cost model decide; 1 = one CTA per tile; 2 = a CTA pair per 256-row tile
  int stream_k;        // tail wave cut into k ranges: 0 = cost model (off when the tile shape is pinned), 1 = on, 2 = off,
                       // 3 = off and one work unit per CTA, dealt out by the hardware block scheduler (for a GEMM
                       // that shares SMs with another stream's kernel)
  // Optional RMSNorm of the result rows: norm_out[M, N] = RMSNorm(D) * norm_w (what the next layer's
  // first GEMM reads). With split-K the reduce pass produces it from the rows it already holds;
  // otherwise the launcher adds a norm launch after the GEMM. Linear epilogue only.
  const void* norm_w;   // [N] bf16, null = no norm
  void* norm_out;       // [M, norm_ld] bf16
  long long norm_ld;
  float norm_eps;
  // Reduce-scatter epilogue: 1 = rows leave through a shared-memory staging piece and one bulk copy per
  // row and 128 columns (256-byte NVLink writes); 0 = 16-byte stores straight from registers.
  int rs_staged;
  // Gated input (all-gather -> GEMM in one pipeline): the rows of A are still being delivered by a
  // collective when the GEMM starts. gate_flags points to this GPU's copy of the collective's row-block
  // flags, [ceil(M/128)][8] words: word [b][r] reaches gate_epoch once rank r has delivered all of its rows
  // of block b (rows 128b .. 128b+127). The TMA producer of a CTA waits (bounded) for the gate_nranks words
  // of an M tile before its first load of that tile, and tiles are walked row block by row block (all
  // column blocks of the first rows first), so the main loops of the first tiles run while the collective
  // is still delivering the later rows. Null = A is complete before the launch. Linear and SwiGLU
  // epilogues; no split-K and no stream-K tail in this mode.
  const unsigned int* gate_flags;
  int gate_epoch, gate_nranks;
} nfk_gemm_params;

int nfk_gemm_bf16(const nfk_gemm_params* p, cudaStream_t stream);

typedef struct nfk_gemm_plan {
  int tile_n, tile_m, cta_group, split_k, stream_k;
  int tiles, workers, num_kb;          // output tiles, CTAs (or CTA pairs), 64-wide k-blocks
  int tail_first_tile, tail_range_kb, tail_max_pieces;   // stream-K tail (tail_range_kb 0 = none)
  int stages, smem_bytes;
} nfk_gemm_plan;
int nfk_gemm_describe(const nfk_gemm_params* p, nfk_gemm_plan* out);

// ------------------------------------------------------------------------------------------------
// Elementwise / normalisation / gather kernels (elementwise.cu)
// ------------------------------------------------------------------------------------------------
// out[r,:] = x[r,:] * rsqrt(mean(x[r,:]^2) + eps) * w[:]
int nfk_rmsnorm(void* out, const void* x, const void* w, int rows, int cols, float eps,
                cudaStream_t stream);
// resid[r,:] += x[r,:]; out[r,:] = rmsnorm(resid[r,:]) (resid updated in place)
int nfk_add_rmsnorm(void* out, void* resid, const void* x, const void* w, int rows, int cols,
                    float eps, cudaStream_t stream);
// Token ids for this iteration, then the embedding rows:
//   id[t] = feedback_src[t] >= 0 ? prev_tokens[feedback_src[t]] : host_ids[t]
//   out[t,:] = table[id[t],:]      (ids outside [0,vocab) are clamped and flagged in status)
// feedback_src / prev_tokens may be null (ids come from host_ids only). ids_out may be null.
int nfk_embedding(void* out, const void* table, const int* host_ids, const int* feedback_src,
                  const int* prev_tokens, int* ids_out, int n_tokens, int hidden, int vocab,
                  unsigned int* status, cudaStream_t stream);
// out[i,:] = in[rows_idx[i],:]
int nfk_gather_rows(void* out, const void* in, const int* rows_idx, int n, int cols, long long ld_in,
                    unsigned int* status, int in_rows, cudaStream_t stream);
// out = silu(gate) * up, elementwise over n elements (n % 8 == 0)
int nfk_silu_mul(void* out, const void* gate, const void* up, long long n, cudaStream_t stream);
// out[r, 0:cols] = in[r, col0 : col0+cols]   (column-block extract / insert with leading dims)
int nfk_copy_cols(void* out, long long ld_out, const void* in, long long ld_in, int rows, int cols,
                  cudaStream_t stream);
// 2-D transpose out[c,r] = in[r,c]
int nfk_transpose(void* out, const void* in, int rows, int cols, cudaStream_t stream);
// Greedy sampler: per row arg-max over `cols` logits. idx_out[r] = col_offset + argmax,
// val_out[r] (optional, fp32) = max. Ties resolve to the lowest index.
int nfk_argmax(int* idx_out, float* val_out, const void* logits, int rows, int cols,
               long long ld, int col_offset, cudaStream_t stream);
// Combine per-shard (val, idx) candidates: cand_val/cand_idx are [shards, rows].
int nfk_argmax_combine(int* idx_out, const float* cand_val, const int* cand_idx, int shards,
                       int rows, cudaStream_t stream);
// Busy-wait for `micros` microseconds (bounded at 1 s); stands in for a collective in ablations.
int nfk_sleep(int micros, cudaStream_t stream);
// Device progress counters: add / clear / bounded wait until *flag >= target.
int nfk_flag_add(unsigned int* flag, unsigned int v, cudaStream_t stream);
int nfk_flag_clear(unsigned int* flag, cudaStream_t stream);
int nfk_flag_wait(const unsigned int* flag, unsigned int target, int timeout_us,
                  unsigned int* status, cudaStream_t stream);

// ------------------------------------------------------------------------------------------------
// RoPE + paged-KV append (rope_append.cu)
// ------------------------------------------------------------------------------------------------
// Paged KV pool of one layer: [num_pages][2 (K,V)][kv_heads][page_size][head_dim] bf16.
typedef struct nfk_rope_append_params {
  const void* qkv;       // [T, ld_qkv] bf16: q at q_off, k at k_off, v at v_off (elements)
  long long ld_qkv;
  int q_off, k_off, v_off;
  void* q_out;           // [T, q_heads*head_dim] rotated queries
  void* kv_pool;         // this layer's pool
  const float* inv_freq; // [head_dim/2] rotary inverse frequencies (any scaling baked in)
  const int* positions;  // [T] absolute position of each token in its sequence
  const int* token_req;  // [T] request index of each token
  const int* kv_indptr;  // [B+1]
  const int* kv_indices; // page ids
  int T, q_heads, kv_heads, head_dim, page_size, num_pages;
  unsigned int* status;
  const float* cos_sin;  // optional [T][head_dim/2][2] (cos, sin) of every token's angles (nfk_rope_table);
                         // null: the kernel computes them itself
} nfk_rope_append_params;
int nfk_rope_append(const nfk_rope_append_params* p, cudaStream_t stream);

// cos / sin of pos[t] * inv_freq[i] for the T tokens of an iteration: every layer rotates by the same
// angles, so they are computed once per iteration instead of once per layer.
typedef struct nfk_rope_table_params {
  float* cos_sin;        // out [T][half][2]
  const float* inv_freq; // [half]
  const int* positions;  // [T]
  int T, half;
} nfk_rope_table_params;
int nfk_rope_table(const nfk_rope_table_params* p, cudaStream_t stream);

// ------------------------------------------------------------------------------------------------
// Attention over the paged KV pool (attention.cu)
// ------------------------------------------------------------------------------------------------
typedef struct nfk_attn_params {
  const void* q;           // [T, q_heads*head_dim] bf16 (rotated)
  void* out;               // [T, q_heads*head_dim] bf16
  const void* kv_pool;     // layer pool, layout above
  const int* qo_indptr;    // [B+1] token range of every request in the dense batch
  const int* kv_indptr;    // [B+1]
  const int* kv_indices;
  const int* kv_last_page_len;  // [B]
  int q_heads, kv_heads, head_dim, page_size, num_pages;
  float sm_scale;
  int num_ctas;            // CTA budget (persistent grid); 0 = one per SM
  // decode: requests [req_begin, req_begin+req_count) each own one query token (qo_indptr[b])
  int req_begin, req_count;
  int chunk_pages;         // split-KV chunk length in pages; 0 = no split
  float* workspace;        // split-KV partials: [req_count*q_heads*max_chunks*(head_dim+2)] fp32
  int max_chunks;
  // prefill: work items (req, first token (global index), token count)
  const int* items;        // [num_items,3]
  int num_items;
  unsigned int* status;
  int decode_stages;       // decode: pages in flight per warp, 3 (0 means 3) or 2 (less shared memory per CTA)
} nfk_attn_params;
int nfk_attn_decode(const nfk_attn_params* p, cudaStream_t stream);
// The same with the pages copied by a TMA producer warp into a ring of decode_stages (2, 3 or 4) pages per
// consumer warp, one work item per warp (attention_dec.cu): full bandwidth from one CTA per SM, for sharing
// SMs with GEMM CTAs. head_dim 128; calls with chunk_pages > 0 are forwarded to nfk_attn_decode.
int nfk_attn_decode_tma(const nfk_attn_params* p, cudaStream_t stream);
int nfk_attn_prefill(const nfk_attn_params* p, cudaStream_t stream);
// Same contract as nfk_attn_prefill for head_dim 128, on tcgen05 tensor cores (attention_tc.cu).
int nfk_attn_prefill_tc(const nfk_attn_params* p, cudaStream_t stream);
// The same on a warp-specialised pipeline: a TMA load warp (whole pages, no transposes), an MMA warp that
// issues the next tile's scores under this tile's softmax, four softmax warps (attention_ws.cu).
int nfk_attn_prefill_ws(const nfk_attn_params* p, cudaStream_t stream);

// ------------------------------------------------------------------------------------------------
// KV offload (kv_offload.cu): gather / scatter whole pages between the pool and a staging buffer
// ------------------------------------------------------------------------------------------------
// page_bytes = 2*kv_heads*page_size*head_dim*2. direction 0: staging[i] = pool[page_ids[i]];
// direction 1: pool[page_ids[i]] = staging[i].
int nfk_kv_move_pages(void* pool, void* staging, const int* page_ids, int n_pages,
                      long long page_bytes, int num_pages, int direction, int num_ctas,
                      unsigned int* status, cudaStream_t stream);

// ------------------------------------------------------------------------------------------------
// Tensor-parallel collectives on a symmetric heap (collectives.cu)
// ------------------------------------------------------------------------------------------------
typedef struct nfk_comm_ctx {
  void* heap[8];       // base of every rank's symmetric heap as mapped into this process
  int rank, nranks;
} nfk_comm_ctx;

typedef struct nfk_allreduce_params {
  nfk_comm_ctx ctx;
  long long buf_off;      // byte offset of the bf16 [rows, ld] buffer inside the heap (summed in place)
  long long flag_off;     // byte offset of this op's 128-byte flag block
  int rows, cols;
  long long ld;           // elements
  int epoch;              // monotonic per call on this flag block (e.g. iteration number)
  int num_ctas;
  const void* norm_w;     // optional: RMSNorm weight [cols]; normed rows go to norm_out on all ranks
  long long norm_out_off; // byte offset of the bf16 [rows, norm_ld] output inside the heap
  long long norm_ld;
  float eps;
  unsigned int* status;
  int push_sum;           // 1: write the sum back into the buffer on every rank (in-place all-reduce)
  const void* resid;      // optional local bf16 [rows, resid_ld]: owned rows are added to the sum
  long long resid_ld;
  void* sum_out;          // optional local bf16 [rows, sum_ld]: owned rows of the sum are stored here
  long long sum_ld;
  int src_mode;           // 0: pull row i from every rank's buffer. 1: the partials were pushed here by a
                          //    NFK_EPI_REDUCE_SCATTER GEMM: owned row k of rank r's partial sits in the local
                          //    slab at buf_off + (r * slab_rows + k) * ld (no NVLink loads, no ready signal)
                          //    2: rank r's buffer holds columns [r*cols/nranks, (r+1)*cols/nranks) of every row (the
                          //    output of an N-split GEMM): an owned row is gathered from the ranks' column blocks
                          //    instead of summed, then residual / norm / pushes as in mode 0
  int slab_rows;
  int wide;               // 1 (8 ranks): twice the loads in flight per phase, the norm pass re-reads the stored sum
  // Optional row-block flags for a consumer that starts before this collective has finished (see
  // nfk_gemm_params::gate_flags): gate_off is the heap offset of [ceil(rows/128)][8] words (same offset on
  // every rank), gate_cnt a local array of ceil(rows/128) zero-initialised words (this rank's rows done per
  // block; reset by the kernel). Once a rank has pushed all the normed rows it owns inside block b it writes
  // `epoch` into word [b][rank] on every rank. Needs norm_w / norm_out (the pushed rows are what is gated).
  long long gate_off;
  unsigned int* gate_cnt;
  // 1: the normed rows this rank owns are stored into its OWN copy of norm_out only and the kernel ends
  // without the exit handshake: the caller delivers them to the peers with copy-engine copies (no SM
  // involved, see parallel/collectives.py) and closes with nfk_comm_barrier. Needs norm_w; no gate flags.
  int push_mode;
  void* mc_heap;          // optional: the heaps' NVLink multicast mapping (one address that stands for the same
                          //    offset on every rank). Non-null selects the in-switch form: owned rows are summed by
                          //    multimem.ld_reduce and results are written to all ranks by multimem.st (src_mode 0 only)
} nfk_allreduce_params;
int nfk_allreduce(const nfk_allreduce_params* p, cudaStream_t stream);

typedef struct nfk_allgather_params {
  nfk_comm_ctx ctx;
  long long buf_off;       // symmetric buffer holding nranks shards, shard r at buf_off + r*shard_stride
  long long shard_bytes, shard_stride, flag_off;
  int epoch, num_ctas, handshake_in;
  unsigned int* status;
  // Column-wise form (rows > 1): the buffer is [rows][...] with row_stride bytes between rows, and
  // rank r owns the shard_bytes starting at byte r*shard_stride of every row (its column block).
  // rows <= 1 is the flat form above.
  int rows;
  long long row_stride;
} nfk_allgather_params;
int nfk_allgather(const nfk_allgather_params* p, cudaStream_t stream);

typedef struct nfk_comm_barrier_params {
  nfk_comm_ctx ctx;
  long long flag_off;
  int epoch;
  unsigned int* status;
} nfk_comm_barrier_params;
int nfk_comm_barrier(const nfk_comm_barrier_params* p, cudaStream_t stream);

// Symmetric heap plumbing: allocate (zero-filled), export / open CUDA IPC handles (64 bytes).
int nfk_symm_alloc(void** out, long long bytes);
int nfk_symm_free(void* p);
int nfk_ipc_get_handle(void* ptr, unsigned char* out64);
int nfk_ipc_open_handle(const unsigned char* in64, void** out);
int nfk_ipc_close_handle(void* p);

// ------------------------------------------------------------------------------------------------
// Uniform launch ABI (abi.cu): every op is also reachable as  int fn(const <params>*, cudaStream_t)
// so that a generic executor can replay a list of (function pointer, parameter block) pairs.
// ------------------------------------------------------------------------------------------------
typedef struct nfk_norm_params {
  void* out; const void* x; const void* w; void* resid;   // resid != NULL: resid += x, out = norm(resid)
  int rows, cols; float eps;
} nfk_norm_params;
typedef struct nfk_embedding_params {
  void* out; const void* table; const int* host_ids; const int* feedback_src; const int* prev_tokens;
  int* ids_out; int n_tokens, hidden, vocab; unsigned int* status;
} nfk_embedding_params;
typedef struct nfk_gather_params {
  void* out; const void* in; const int* rows_idx; int n, cols; long long ld_in; int in_rows;
  unsigned int* status;
} nfk_gather_params;
typedef struct nfk_argmax_params {
  int* idx_out; float* val_out; const void* logits; int rows, cols; long long ld; int col_offset;
} nfk_argmax_params;
typedef struct nfk_argmax_combine_params {
  int* idx_out; const float* cand_val; const int* cand_idx; int shards, rows;
} nfk_argmax_combine_params;
typedef struct nfk_copy_cols_params {
  void* out; long long ld_out; const void* in; long long ld_in; int rows, cols;
} nfk_copy_cols_params;
typedef struct nfk_memcpy_params {   // plain async copy (any direction); elem_bytes * count bytes
  void* dst; const void* src; long long elem_bytes; int count;
} nfk_memcpy_params;
typedef struct nfk_memcpy2d_params {  // strided async copy: `height` rows of `width` bytes, row pitches in bytes
  void* dst; const void* src; long long dpitch, spitch, width; int height;
} nfk_memcpy2d_params;
typedef struct nfk_kv_move_params {
  void* pool; void* staging; const int* page_ids; int n_pages; long long page_bytes; int num_pages;
  int direction; int num_ctas; unsigned int* status;
} nfk_kv_move_params;

int nfk_norm_p(const nfk_norm_params* p, cudaStream_t s);
int nfk_embedding_p(const nfk_embedding_params* p, cudaStream_t s);
int nfk_gather_p(const nfk_gather_params* p, cudaStream_t s);
int nfk_argmax_p(const nfk_argmax_params* p, cudaStream_t s);
int nfk_argmax_combine_p(const nfk_argmax_combine_params* p, cudaStream_t s);
int nfk_copy_cols_p(const nfk_copy_cols_params* p, cudaStream_t s);
int nfk_memcpy_p(const nfk_memcpy_params* p, cudaStream_t s);
typedef struct nfk_sleep_params { int micros; } nfk_sleep_params;   // nfk_sleep as an op of the graph
int nfk_sleep_p(const nfk_sleep_params* p, cudaStream_t s);
int nfk_kv_move_p(const nfk_kv_move_params* p, cudaStream_t s);

#ifdef __cplusplus
}
#endif
