// Uniform launch ABI: thin `int fn(const params*, cudaStream_t)` forms of the entry points that take
// scalar arguments, so an executor can store (function pointer, parameter block) pairs and replay
// them without knowing any kernel's signature.
#include "common.cuh"
#include "kernels.h"

using namespace nf;

extern "C" int nfk_norm_p(const nfk_norm_params* p, cudaStream_t s) {
  if (!p) return NF_ERR_BAD_ARG;
  return p->resid ? nfk_add_rmsnorm(p->out, p->resid, p->x, p->w, p->rows, p->cols, p->eps, s)
                  : nfk_rmsnorm(p->out, p->x, p->w, p->rows, p->cols, p->eps, s);
}
extern "C" int nfk_embedding_p(const nfk_embedding_params* p, cudaStream_t s) {
  if (!p) return NF_ERR_BAD_ARG;
  return nfk_embedding(p->out, p->table, p->host_ids, p->feedback_src, p->prev_tokens, p->ids_out,
                       p->n_tokens, p->hidden, p->vocab, p->status, s);
}
extern "C" int nfk_gather_p(const nfk_gather_params* p, cudaStream_t s) {
  if (!p) return NF_ERR_BAD_ARG;
  return nfk_gather_rows(p->out, p->in, p->rows_idx, p->n, p->cols, p->ld_in, p->status, p->in_rows, s);
}
extern "C" int nfk_argmax_p(const nfk_argmax_params* p, cudaStream_t s) {
  if (!p) return NF_ERR_BAD_ARG;
  return nfk_argmax(p->idx_out, p->val_out, p->logits, p->rows, p->cols, p->ld, p->col_offset, s);
}
extern "C" int nfk_argmax_combine_p(const nfk_argmax_combine_params* p, cudaStream_t s) {
  if (!p) return NF_ERR_BAD_ARG;
  return nfk_argmax_combine(p->idx_out, p->cand_val, p->cand_idx, p->shards, p->rows, s);
}
extern "C" int nfk_copy_cols_p(const nfk_copy_cols_params* p, cudaStream_t s) {
  if (!p) return NF_ERR_BAD_ARG;
  return nfk_copy_cols(p->out, p->ld_out, p->in, p->ld_in, p->rows, p->cols, s);
}
extern "C" int nfk_memcpy_p(const nfk_memcpy_params* p, cudaStream_t s) {
  if (!p || p->count < 0 || p->elem_bytes < 0) return NF_ERR_BAD_ARG;
  const long long bytes = p->elem_bytes * p->count;
  if (bytes == 0) return NF_OK;
  if (!p->dst || !p->src) return NF_ERR_BAD_ARG;
  return cudaMemcpyAsync(p->dst, p->src, static_cast<size_t>(bytes), cudaMemcpyDefault, s) == cudaSuccess
             ? NF_OK : NF_ERR_CUDA;
}
extern "C" int nfk_memcpy2d_p(const nfk_memcpy2d_params* p, cudaStream_t s) {
  if (!p || p->height < 0 || p->width < 0 || p->dpitch < p->width || p->spitch < p->width) return NF_ERR_BAD_ARG;
  if (p->height == 0 || p->width == 0) return NF_OK;
  if (!p->dst || !p->src) return NF_ERR_BAD_ARG;
  return cudaMemcpy2DAsync(p->dst, static_cast<size_t>(p->dpitch), p->src, static_cast<size_t>(p->spitch),
                           static_cast<size_t>(p->width), static_cast<size_t>(p->height), cudaMemcpyDefault,
                           s) == cudaSuccess
             ? NF_OK : NF_ERR_CUDA;
}
extern "C" int nfk_sleep_p(const nfk_sleep_params* p, cudaStream_t s) {
  if (!p) return NF_ERR_BAD_ARG;
  return p->micros == 0 ? NF_OK : nfk_sleep(p->micros, s);
}
extern "C" int nfk_kv_move_p(const nfk_kv_move_params* p, cudaStream_t s) {
  if (!p) return NF_ERR_BAD_ARG;
  return nfk_kv_move_pages(p->pool, p->staging, p->page_ids, p->n_pages, p->page_bytes, p->num_pages,
                           p->direction, p->num_ctas, p->status, s);
}
