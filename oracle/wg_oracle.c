/*
 * CPU oracle for the WholeGraph embedding hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, what the reference's CUDA kernels and its test-side CPU
 * optimizer compute, so that the sm_100a kernels of this repository can be checked against
 * it.  It is linked or loaded only by the tests, the smoke check and the CPU-baseline leg of
 * the benchmark; the product library never calls it.
 *
 * Parity pin: the reference has no CPU implementation of gather / scatter, cannot be run
 * in a GPU-less container, and ships no golden byte vectors (its tests draw unseeded random
 * indices).  The oracle is therefore pinned against (1) the closed-form table generators and
 * bitwise expectations of the reference's own tests, re-evaluated in tests/test_oracle_pins.py,
 * (2) numpy's IEEE fp16 conversion for every fp32 exponent class, and (3) on a GPU box, the
 * reference's own kernels compiled from their sources (oracle/ref_kernels.cu).
 *
 * Each function cites the reference file:line it follows (paths relative to the reference
 * repository root).
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* dtype codes = wholegraph_dtype_t, cpp/include/wholegraph/tensor_description.h:18-29 */
enum {
  DT_UNKNOWN = 0,
  DT_FLOAT   = 1,
  DT_HALF    = 2,
  DT_DOUBLE  = 3,
  DT_BF16    = 4,
  DT_INT     = 5,
  DT_INT64   = 6,
  DT_INT16   = 7,
  DT_INT8    = 8
};

/* cpp/src/wholegraph/tensor_description.cpp:11-27 */
int64_t wgo_dtype_size(int dt)
{
  switch (dt) {
    case DT_INT8: return 1;
    case DT_INT16:
    case DT_BF16:
    case DT_HALF: return 2;
    case DT_INT:
    case DT_FLOAT: return 4;
    case DT_INT64:
    case DT_DOUBLE: return 8;
    default: return 0;
  }
}

static int is_float_dt(int dt)
{
  return dt == DT_FLOAT || dt == DT_HALF || dt == DT_DOUBLE || dt == DT_BF16;
}
static int is_int_dt(int dt)
{
  return dt == DT_INT || dt == DT_INT64 || dt == DT_INT16 || dt == DT_INT8;
}

/* ---------------------------------------------------------------------------------------
 * Scalar conversions.  The reference casts with static_cast on device
 * (cpp/src/wholegraph_tensor_ops/functions/gather_scatter_func.cuh:150-197): anything that
 * touches fp16 / bf16 goes through fp32, and fp32 -> fp16 / bf16 is round-to-nearest-even
 * with NaN mapped to 0x7FFF.
 * ------------------------------------------------------------------------------------- */
static inline uint32_t f2u(float f)
{
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
}
static inline float u2f(uint32_t u)
{
  float f;
  memcpy(&f, &u, 4);
  return f;
}

uint16_t wgo_float_to_half(float f)
{
  uint32_t x    = f2u(f);
  uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t abs_ = x & 0x7FFFFFFFu;
  if (abs_ > 0x7F800000u) return 0x7FFFu;                    /* NaN -> canonical */
  if (abs_ >= 0x47800000u) {                                 /* >= 65536: overflow or inf */
    return (uint16_t)(sign | 0x7C00u);
  }
  if (abs_ >= 0x38800000u) { /* normal half range: exponent >= -14 */
    uint32_t mant = abs_ & 0x007FFFFFu;
    uint32_t exp_ = (abs_ >> 23) - 112u; /* rebias 127 -> 15 */
    uint32_t h    = (exp_ << 10) | (mant >> 13);
    uint32_t rem  = mant & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) h++; /* may carry into exponent / inf */
    return (uint16_t)(sign | h);
  }
  if (abs_ < 0x33000000u) return (uint16_t)sign; /* < 2^-25: rounds to zero */
  {
    /* subnormal half: value = mant24 * 2^(e-150); half subnormal unit = 2^-24 */
    uint32_t e      = abs_ >> 23;
    uint32_t mant24 = (abs_ & 0x007FFFFFu) | 0x00800000u;
    uint32_t shift  = 126u - e; /* 14..24 */
    uint32_t h      = mant24 >> shift;
    uint32_t rem    = mant24 & ((1u << shift) - 1u);
    uint32_t half_  = 1u << (shift - 1u);
    if (rem > half_ || (rem == half_ && (h & 1u))) h++;
    return (uint16_t)(sign | h);
  }
}

float wgo_half_to_float(uint16_t h)
{
  uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
  uint32_t exp_ = (h >> 10) & 0x1Fu;
  uint32_t mant = h & 0x3FFu;
  if (exp_ == 0x1Fu) return u2f(sign | 0x7F800000u | (mant << 13));
  if (exp_ != 0) return u2f(sign | ((exp_ + 112u) << 23) | (mant << 13));
  if (mant == 0) return u2f(sign);
  {
    /* subnormal: normalise */
    int e = -1;
    do {
      e++;
      mant <<= 1;
    } while ((mant & 0x400u) == 0);
    return u2f(sign | ((uint32_t)(112 - e) << 23) | ((mant & 0x3FFu) << 13));
  }
}

uint16_t wgo_float_to_bf16(float f)
{
  uint32_t x = f2u(f);
  if ((x & 0x7FFFFFFFu) > 0x7F800000u) return 0x7FFFu; /* NaN -> canonical */
  x += 0x7FFFu + ((x >> 16) & 1u);                     /* round to nearest even */
  return (uint16_t)(x >> 16);
}

float wgo_bf16_to_float(uint16_t b) { return u2f((uint32_t)b << 16); }

/* Load one element as the "wide" value the reference's type_caster would produce. */
static inline double load_float_elt(const void* p, int dt, int64_t i)
{
  switch (dt) {
    case DT_FLOAT: return (double)((const float*)p)[i];
    case DT_DOUBLE: return ((const double*)p)[i];
    case DT_HALF: return (double)wgo_half_to_float(((const uint16_t*)p)[i]);
    default: return (double)wgo_bf16_to_float(((const uint16_t*)p)[i]);
  }
}
/* Store with the reference's rounding chain: double -> float (RN) -> half / bf16 (RN). */
static inline void store_float_elt(void* p, int dt, int64_t i, double v)
{
  switch (dt) {
    case DT_FLOAT: ((float*)p)[i] = (float)v; break;
    case DT_DOUBLE: ((double*)p)[i] = v; break;
    case DT_HALF: ((uint16_t*)p)[i] = wgo_float_to_half((float)v); break;
    default: ((uint16_t*)p)[i] = wgo_float_to_bf16((float)v); break;
  }
}
static inline int64_t load_int_elt(const void* p, int dt, int64_t i)
{
  switch (dt) {
    case DT_INT8: return ((const int8_t*)p)[i];
    case DT_INT16: return ((const int16_t*)p)[i];
    case DT_INT: return ((const int32_t*)p)[i];
    default: return ((const int64_t*)p)[i];
  }
}
static inline void store_int_elt(void* p, int dt, int64_t i, int64_t v)
{
  switch (dt) {
    case DT_INT8: ((int8_t*)p)[i] = (int8_t)(uint8_t)(uint64_t)v; break;
    case DT_INT16: ((int16_t*)p)[i] = (int16_t)(uint16_t)(uint64_t)v; break;
    case DT_INT: ((int32_t*)p)[i] = (int32_t)(uint32_t)(uint64_t)v; break;
    default: ((int64_t*)p)[i] = v; break;
  }
}

/* Copy `dim` elements with the cast the reference applies (gather_scatter_func.cuh:193-197). */
static void copy_cast_row(void* dst, int dst_dt, int64_t dst_elt, const void* src, int src_dt,
                          int64_t src_elt, int64_t dim)
{
  if (dst_dt == src_dt) {
    int64_t es = wgo_dtype_size(dst_dt);
    memcpy((char*)dst + dst_elt * es, (const char*)src + src_elt * es, (size_t)(dim * es));
    return;
  }
  if (is_float_dt(src_dt)) {
    if (src_dt == DT_FLOAT && dst_dt == DT_HALF) { /* fast common case */
      const float* s = (const float*)src + src_elt;
      uint16_t* d    = (uint16_t*)dst + dst_elt;
      for (int64_t c = 0; c < dim; c++) d[c] = wgo_float_to_half(s[c]);
      return;
    }
    if (src_dt == DT_FLOAT && dst_dt == DT_BF16) {
      const float* s = (const float*)src + src_elt;
      uint16_t* d    = (uint16_t*)dst + dst_elt;
      for (int64_t c = 0; c < dim; c++) d[c] = wgo_float_to_bf16(s[c]);
      return;
    }
    for (int64_t c = 0; c < dim; c++)
      store_float_elt(dst, dst_dt, dst_elt + c, load_float_elt(src, src_dt, src_elt + c));
  } else {
    for (int64_t c = 0; c < dim; c++)
      store_int_elt(dst, dst_dt, dst_elt + c, load_int_elt(src, src_dt, src_elt + c));
  }
}

static inline int64_t load_index(const void* idx, int idx_dt, int64_t i)
{
  return idx_dt == DT_INT ? (int64_t)((const int32_t*)idx)[i] : ((const int64_t*)idx)[i];
}

/* ---------------------------------------------------------------------------------------
 * Thread helper: split [0, n) over nthreads like the reference test's MultiThreadRun
 * (cpp/tests/wholegraph_tensor_ops/wholegraph_embedding_gradient_apply_tests.cu:396-401).
 * ------------------------------------------------------------------------------------- */
typedef void (*range_fn_t)(void* ctx, int64_t begin, int64_t end);
typedef struct {
  range_fn_t fn;
  void* ctx;
  int64_t begin, end;
} range_job_t;
static void* range_trampoline(void* p)
{
  range_job_t* j = (range_job_t*)p;
  j->fn(j->ctx, j->begin, j->end);
  return NULL;
}
static void parallel_for(int nthreads, int64_t n, range_fn_t fn, void* ctx)
{
  if (nthreads <= 1 || n < 2) {
    fn(ctx, 0, n);
    return;
  }
  if (nthreads > 256) nthreads = 256;
  pthread_t th[256];
  range_job_t jobs[256];
  for (int t = 0; t < nthreads; t++) {
    jobs[t].fn    = fn;
    jobs[t].ctx   = ctx;
    jobs[t].begin = n * t / nthreads;
    jobs[t].end   = n * (t + 1) / nthreads;
    pthread_create(&th[t], NULL, range_trampoline, &jobs[t]);
  }
  for (int t = 0; t < nthreads; t++) pthread_join(th[t], NULL);
}

/* ---------------------------------------------------------------------------------------
 * Gather: gather_func_kernel, gather_scatter_func.cuh:278-303.
 *   out[out_off + out_row*out_stride + c] = cast(table[tab_off + idx*tab_stride + c])
 *   out_row = raw_pos[i] if raw_pos != NULL else i;  idx < 0 -> row skipped.
 * Returns 0, or -1 for an illegal dtype pair (gather_func.cu:63-70).
 * ------------------------------------------------------------------------------------- */
typedef struct {
  const void* table;
  int tab_dt;
  int64_t dim, tab_stride, tab_off;
  const void* idx;
  int idx_dt;
  const int64_t* raw_pos;
  void* out;
  int out_dt;
  int64_t out_stride, out_off;
} gather_ctx_t;

static void gather_range(void* p, int64_t b, int64_t e)
{
  gather_ctx_t* g = (gather_ctx_t*)p;
  for (int64_t i = b; i < e; i++) {
    int64_t id = load_index(g->idx, g->idx_dt, i);
    if (id < 0) continue;
    int64_t orow = g->raw_pos ? g->raw_pos[i] : i;
    copy_cast_row(g->out, g->out_dt, g->out_off + orow * g->out_stride, g->table, g->tab_dt,
                  g->tab_off + id * g->tab_stride, g->dim);
  }
}

int wgo_gather(const void* table, int tab_dt, int64_t dim, int64_t tab_stride, int64_t tab_off,
               const void* idx, int idx_dt, int64_t n, const int64_t* raw_pos, void* out,
               int out_dt, int64_t out_stride, int64_t out_off, int nthreads)
{
  if (!((is_float_dt(tab_dt) && is_float_dt(out_dt)) || (is_int_dt(tab_dt) && is_int_dt(out_dt))))
    return -1;
  if (n == 0 || dim == 0) return 0;
  gather_ctx_t g = {table, tab_dt, dim, tab_stride, tab_off, idx, idx_dt,
                    raw_pos, out, out_dt, out_stride, out_off};
  parallel_for(nthreads, n, gather_range, &g);
  return 0;
}

/* ---------------------------------------------------------------------------------------
 * Scatter: scatter_func_kernel, gather_scatter_func.cuh:548-585.
 *   table[tab_off + idx*tab_stride + c] = cast(in[in_off + i*in_stride + c]);  idx < 0 skipped.
 * Rows are written in ascending i, so with duplicate indices the LAST writer wins here; the
 * device kernels give no such guarantee, and parity tests use unique indices.
 * ------------------------------------------------------------------------------------- */
typedef struct {
  const void* in;
  int in_dt;
  int64_t dim, in_stride, in_off;
  const void* idx;
  int idx_dt;
  void* table;
  int tab_dt;
  int64_t tab_stride, tab_off;
} scatter_ctx_t;

static void scatter_range(void* p, int64_t b, int64_t e)
{
  scatter_ctx_t* s = (scatter_ctx_t*)p;
  for (int64_t i = b; i < e; i++) {
    int64_t id = load_index(s->idx, s->idx_dt, i);
    if (id < 0) continue;
    copy_cast_row(s->table, s->tab_dt, s->tab_off + id * s->tab_stride, s->in, s->in_dt,
                  s->in_off + i * s->in_stride, s->dim);
  }
}

int wgo_scatter(const void* in, int in_dt, int64_t dim, int64_t in_stride, int64_t in_off,
                const void* idx, int idx_dt, int64_t n, void* table, int tab_dt,
                int64_t tab_stride, int64_t tab_off, int nthreads)
{
  if (!((is_float_dt(tab_dt) && is_float_dt(in_dt)) || (is_int_dt(tab_dt) && is_int_dt(in_dt))))
    return -1;
  if (n == 0 || dim == 0) return 0;
  scatter_ctx_t s = {in, in_dt, dim, in_stride, in_off, idx, idx_dt,
                     table, tab_dt, tab_stride, tab_off};
  parallel_for(nthreads, n, scatter_range, &s);
  return 0;
}

/* ---------------------------------------------------------------------------------------
 * Partition: default split ceil(rows / W) rows per rank, last ranks short or empty
 * (cpp/src/wholegraph/memory_handle.cpp:1241-1262, :1609-1615).  offsets has W + 1 entries.
 * ------------------------------------------------------------------------------------- */
void wgo_equal_partition_offsets(int64_t rows, int world, int64_t* offsets)
{
  int64_t per = (rows + world - 1) / world;
  for (int r = 0; r < world; r++) {
    int64_t s  = (int64_t)r * per;
    offsets[r] = s < rows ? s : rows;
  }
  offsets[world] = rows;
}

/* Owner of an id = the last rank whose first row is <= id
 * (cpp/src/wholegraph_tensor_ops/functions/bucket_ids_func.cu:21-38). */
int wgo_owner(int64_t id, const int64_t* offsets, int world)
{
  int r = world - 1;
  while (r > 0 && offsets[r] > id) r--;
  return r;
}

/* ---------------------------------------------------------------------------------------
 * Bucket-and-sort of one rank's request list
 * (cpp/src/wholegraph_tensor_ops/functions/exchange_ids_nccl_func.cu:32-104, :146-215):
 * stable sort of (id, position) by id as UNSIGNED keys, so negatives go to the tail and are
 * excluded from the per-owner counts (bucket_ids_func.cu:62).
 *   counts[W]      ids sent to each owner
 *   sorted_ids[n]  ids in send order (first sum(counts) entries are valid)
 *   raw_pos[n]     original position of each sorted id
 * ------------------------------------------------------------------------------------- */
typedef struct {
  uint64_t key;
  int64_t pos;
} kp_t;
static int kp_cmp(const void* a, const void* b)
{
  const kp_t* x = (const kp_t*)a;
  const kp_t* y = (const kp_t*)b;
  if (x->key != y->key) return x->key < y->key ? -1 : 1;
  return x->pos < y->pos ? -1 : (x->pos > y->pos ? 1 : 0);
}

int wgo_bucket_sort_ids(const void* idx, int idx_dt, int64_t n, const int64_t* offsets, int world,
                        int64_t* counts, int64_t* sorted_ids, int64_t* raw_pos)
{
  kp_t* kp = (kp_t*)malloc(sizeof(kp_t) * (size_t)(n > 0 ? n : 1));
  if (!kp) return -1;
  for (int r = 0; r < world; r++) counts[r] = 0;
  for (int64_t i = 0; i < n; i++) {
    int64_t id = load_index(idx, idx_dt, i);
    kp[i].key  = (uint64_t)id;
    kp[i].pos  = i;
    if (id >= 0) counts[wgo_owner(id, offsets, world)]++;
  }
  qsort(kp, (size_t)n, sizeof(kp_t), kp_cmp); /* (key, pos) order == stable sort by key */
  for (int64_t i = 0; i < n; i++) {
    sorted_ids[i] = (int64_t)kp[i].key;
    raw_pos[i]    = kp[i].pos;
  }
  free(kp);
  return 0;
}

/* ---------------------------------------------------------------------------------------
 * Duplicate-gradient sum (cpp/src/wholegraph_tensor_ops/functions/
 * exchange_embeddings_nccl_func.cu:68-95, :127-151): stable sort by id, then for each distinct
 * id add its gradient rows one after the other, in arrival order, in fp32.
 *   uniq_ids[n], uniq_grads[n*dim] are filled for the first `return value` entries.
 * grads rows are `grad_stride` elements apart; grad dtype fp32 / fp16 / bf16.
 * `block` = 0 restates the reference (one chain per id).  `block` > 0 restates what this
 * repository's kernels do for ids that occur more than `block` times: the run is cut into blocks
 * of `block` rows in arrival order, each block is summed in order, and the block sums are added
 * in block order.
 * ------------------------------------------------------------------------------------- */
int64_t wgo_dedup_gradients_blocked(const void* idx, int idx_dt, int64_t n, const void* grads,
                                    int grad_dt, int64_t dim, int64_t grad_stride, int64_t block,
                                    int64_t* uniq_ids, float* uniq_grads)
{
  if (n == 0) return 0;
  kp_t* kp = (kp_t*)malloc(sizeof(kp_t) * (size_t)n);
  float* part = (float*)malloc(sizeof(float) * (size_t)(dim > 0 ? dim : 1));
  if (!kp || !part) return -1;
  for (int64_t i = 0; i < n; i++) {
    kp[i].key = (uint64_t)load_index(idx, idx_dt, i);
    kp[i].pos = i;
  }
  qsort(kp, (size_t)n, sizeof(kp_t), kp_cmp);
  int64_t u = 0;
  for (int64_t first = 0; first < n;) {
    int64_t last = first + 1;
    while (last < n && kp[last].key == kp[first].key) last++;
    uniq_ids[u] = (int64_t)kp[first].key;
    float* acc  = uniq_grads + u * dim;
    int64_t len = last - first;
    /* block == 0 or a short run: one chain, the reference's order */
    int64_t step = (block > 0 && len > block) ? block : len;
    for (int64_t b = first; b < last; b += step) {
      int64_t e = b + step < last ? b + step : last;
      for (int64_t i = b; i < e; i++) {
        for (int64_t c = 0; c < dim; c++) {
          float g = (float)load_float_elt(grads, grad_dt, kp[i].pos * grad_stride + c);
          if (i == b)
            part[c] = g;
          else
            part[c] += g;
        }
      }
      for (int64_t c = 0; c < dim; c++) {
        if (b == first)
          acc[c] = part[c];
        else
          acc[c] += part[c];
      }
    }
    u++;
    first = last;
  }
  free(kp);
  free(part);
  return u;
}

int64_t wgo_dedup_gradients(const void* idx, int idx_dt, int64_t n, const void* grads, int grad_dt,
                            int64_t dim, int64_t grad_stride, int64_t* uniq_ids, float* uniq_grads)
{
  return wgo_dedup_gradients_blocked(idx, idx_dt, n, grads, grad_dt, dim, grad_stride, 0, uniq_ids,
                                     uniq_grads);
}

/* ---------------------------------------------------------------------------------------
 * Sparse optimizers.  Arithmetic and operation order follow the reference kernels
 * (cpp/src/wholegraph_tensor_ops/functions/embedding_optimizer_func.cu:203-214 SGD, :386-421
 * Lazy Adam, :655-671 AdaGrad, :865-881 RMSProp) and its CPU test optimizer
 * (cpp/tests/wholegraph_tensor_ops/wholegraph_embedding_gradient_apply_tests.cu:170-380).
 * Every product and sum is a separately rounded fp32 operation (this file is compiled with
 * -ffp-contract=off).
 *
 * `ids` are global row ids, already unique; row = ids[i] - local_start indexes the local shard.
 * weights: dtype w_dt (fp32 / fp16 / bf16), rows `w_stride` elements apart.
 * state  : fp32 rows `state_stride` elements apart; Lazy Adam keeps m at [0, dim) and v at
 *          [w_stride_padded, w_stride_padded + dim) of the same row
 *          (embedding_optimizer_func.cu:386-387: v_ptr = m_ptr + local_embedding_stride).
 * beta12t: fp32 [rows, 2], running beta1^t, beta2^t per ROW, multiplied on every touch.
 * ------------------------------------------------------------------------------------- */
enum { OPT_SGD = 1, OPT_LAZY_ADAM = 2, OPT_RMSPROP = 3, OPT_ADAGRAD = 4 };

typedef struct {
  int opt;
  const int64_t* ids;
  const float* grads;
  int64_t dim, grad_stride;
  void* w;
  int w_dt;
  int64_t w_stride;
  float* state;
  int64_t state_stride, v_offset;
  float* beta12t;
  int64_t local_start;
  float lr, weight_decay, epsilon, beta1, beta2, alpha;
  int adam_w;
} opt_ctx_t;

static inline float load_w(const void* w, int dt, int64_t i)
{
  if (dt == DT_FLOAT) return ((const float*)w)[i];
  if (dt == DT_HALF) return wgo_half_to_float(((const uint16_t*)w)[i]);
  return wgo_bf16_to_float(((const uint16_t*)w)[i]);
}
static inline void store_w(void* w, int dt, int64_t i, float v)
{
  if (dt == DT_FLOAT)
    ((float*)w)[i] = v;
  else if (dt == DT_HALF)
    ((uint16_t*)w)[i] = wgo_float_to_half(v);
  else
    ((uint16_t*)w)[i] = wgo_float_to_bf16(v);
}

static void opt_range(void* p, int64_t b, int64_t e)
{
  opt_ctx_t* o = (opt_ctx_t*)p;
  for (int64_t i = b; i < e; i++) {
    int64_t row    = o->ids[i] - o->local_start;
    const float* g = o->grads + i * o->grad_stride;
    int64_t wbase  = row * o->w_stride;
    float* st      = o->state ? o->state + row * o->state_stride : NULL;
    float beta1t = 0.f, beta2t = 0.f;
    if (o->opt == OPT_LAZY_ADAM) {
      beta1t                  = o->beta12t[row * 2 + 0] * o->beta1;
      beta2t                  = o->beta12t[row * 2 + 1] * o->beta2;
      o->beta12t[row * 2 + 0] = beta1t;
      o->beta12t[row * 2 + 1] = beta2t;
    }
    for (int64_t c = 0; c < o->dim; c++) {
      float grad = g[c];
      float w    = load_w(o->w, o->w_dt, wbase + c);
      switch (o->opt) {
        case OPT_SGD: {
          grad += o->weight_decay * w;
          w -= o->lr * grad;
          break;
        }
        case OPT_LAZY_ADAM: {
          if (o->adam_w)
            w -= o->lr * o->weight_decay * w;
          else
            grad = grad + o->weight_decay * w;
          float m    = st[c];
          float v    = st[o->v_offset + c];
          m          = o->beta1 * m + (1 - o->beta1) * grad;
          v          = o->beta2 * v + (1 - o->beta2) * grad * grad;
          float mhat = m / (1 - beta1t);
          float vhat = v / (1 - beta2t);
          w          = w - o->lr * mhat / (sqrtf(vhat) + o->epsilon);
          st[c]      = m;
          st[o->v_offset + c] = v;
          break;
        }
        case OPT_ADAGRAD: {
          grad    = grad + o->weight_decay * w;
          float s = st[c];
          s       = s + grad * grad;
          w       = w - o->lr * grad / (sqrtf(s) + o->epsilon);
          st[c]   = s;
          break;
        }
        default: { /* RMSProp */
          grad    = grad + o->weight_decay * w;
          float v = st[c];
          v       = o->alpha * v + (1 - o->alpha) * grad * grad;
          w       = w - o->lr * grad / (sqrtf(v) + o->epsilon);
          st[c]   = v;
          break;
        }
      }
      store_w(o->w, o->w_dt, wbase + c, w);
    }
  }
}

int wgo_optimizer_apply(int opt, const int64_t* ids, int64_t n, const float* grads, int64_t dim,
                        int64_t grad_stride, void* w, int w_dt, int64_t w_stride, float* state,
                        int64_t state_stride, int64_t v_offset, float* beta12t, int64_t local_start,
                        float lr, float weight_decay, float epsilon, float beta1, float beta2,
                        float alpha, int adam_w, int nthreads)
{
  if (w_dt != DT_FLOAT && w_dt != DT_HALF && w_dt != DT_BF16) return -1;
  opt_ctx_t o = {opt, ids, grads, dim, grad_stride, w, w_dt, w_stride, state, state_stride,
                 v_offset, beta12t, local_start, lr, weight_decay, epsilon, beta1, beta2, alpha,
                 adam_w};
  parallel_for(nthreads, n, opt_range, &o); /* ids are unique: rows are independent */
  return 0;
}

/* ---------------------------------------------------------------------------------------
 * Round-robin id remap, restated literally from storage_idx2wg_emb_idx_kernel
 * (cpp/src/wholegraph_tensor_ops/functions/map_indices_func.cu:16-34): with blocks of `rr`
 * consecutive ids dealt to the W ranks in turn, id -> entry_start + rr * (block / W) + id % rr,
 * where entry_start is the first row of the CALLING rank's shard (:76-78).  The rank the block
 * was dealt to does not enter the result.
 * ------------------------------------------------------------------------------------- */
void wgo_round_robin_map(const void* idx, int idx_dt, int64_t n, int64_t rr, int world,
                         int64_t entry_start, void* out)
{
  for (int64_t i = 0; i < n; i++) {
    int64_t id     = load_index(idx, idx_dt, i);
    int64_t block  = id / rr;
    int64_t mapped = entry_start + rr * (block / world) + id % rr;
    if (idx_dt == DT_INT)
      ((int32_t*)out)[i] = (int32_t)mapped;
    else
      ((int64_t*)out)[i] = mapped;
  }
}
