// Descriptor arithmetic of the C ABI. Behaviour follows the reference's
// cpp/src/wholegraph/tensor_description.cpp:11-226 (sizes, strides and offsets in elements).
#include <wholegraph/global_reference.h>
#include <wholegraph/tensor_description.h>

extern "C" {

size_t wholegraph_dtype_get_element_size(wholegraph_dtype_t dtype)
{
  static const size_t kSize[WHOLEGRAPH_DT_COUNT] = {0, 4, 2, 8, 2, 4, 8, 2, 1};
  if (dtype < WHOLEGRAPH_DT_UNKNOWN || dtype >= WHOLEGRAPH_DT_COUNT) return static_cast<size_t>(-1);
  return kSize[dtype];
}

bool wholegraph_dtype_is_floating_number(wholegraph_dtype_t dtype)
{
  return dtype == WHOLEGRAPH_DT_FLOAT || dtype == WHOLEGRAPH_DT_HALF ||
         dtype == WHOLEGRAPH_DT_DOUBLE || dtype == WHOLEGRAPH_DT_BF16;
}

bool wholegraph_dtype_is_integer_number(wholegraph_dtype_t dtype)
{
  return dtype == WHOLEGRAPH_DT_INT || dtype == WHOLEGRAPH_DT_INT64 ||
         dtype == WHOLEGRAPH_DT_INT16 || dtype == WHOLEGRAPH_DT_INT8;
}

wholegraph_array_description_t wholegraph_create_array_desc(int64_t size,
                                                              int64_t storage_offset,
                                                              wholegraph_dtype_t dtype)
{
  wholegraph_array_description_t d;
  d.size           = size;
  d.storage_offset = storage_offset;
  d.dtype          = dtype;
  return d;
}

wholegraph_matrix_description_t wholegraph_create_matrix_desc(int64_t sizes[2],
                                                                int64_t stride,
                                                                int64_t storage_offset,
                                                                wholegraph_dtype_t dtype)
{
  wholegraph_matrix_description_t d;
  d.sizes[0]       = sizes[0];
  d.sizes[1]       = sizes[1];
  d.stride         = stride;
  d.storage_offset = storage_offset;
  d.dtype          = dtype;
  return d;
}

void wholegraph_initialize_tensor_desc(wholegraph_tensor_description_t* t)
{
  t->dim = 0;
  for (int i = 0; i < WHOLEGRAPH_MAX_TENSOR_DIM; i++) t->sizes[i] = t->strides[i] = 1;
  t->storage_offset = 0;
  t->dtype          = WHOLEGRAPH_DT_UNKNOWN;
}

void wholegraph_copy_array_desc_to_matrix(wholegraph_matrix_description_t* m,
                                           wholegraph_array_description_t* a)
{
  m->sizes[0]       = a->size;
  m->sizes[1]       = 1;
  m->stride         = 1;
  m->storage_offset = a->storage_offset;
  m->dtype          = a->dtype;
}

void wholegraph_copy_array_desc_to_tensor(wholegraph_tensor_description_t* t,
                                           wholegraph_array_description_t* a)
{
  wholegraph_initialize_tensor_desc(t);
  t->dim            = 1;
  t->sizes[0]       = a->size;
  t->strides[0]     = 1;
  t->storage_offset = a->storage_offset;
  t->dtype          = a->dtype;
}

void wholegraph_copy_matrix_desc_to_tensor(wholegraph_tensor_description_t* t,
                                            wholegraph_matrix_description_t* m)
{
  wholegraph_initialize_tensor_desc(t);
  t->dim            = 2;
  t->sizes[0]       = m->sizes[0];
  t->sizes[1]       = m->sizes[1];
  t->strides[0]     = m->stride;
  t->strides[1]     = 1;
  t->storage_offset = m->storage_offset;
  t->dtype          = m->dtype;
}

static bool known_dtype(wholegraph_dtype_t dt)
{
  return dt > WHOLEGRAPH_DT_UNKNOWN && dt < WHOLEGRAPH_DT_COUNT;
}

bool wholegraph_convert_tensor_desc_to_array(wholegraph_array_description_t* a,
                                              wholegraph_tensor_description_t* t)
{
  if (!known_dtype(t->dtype) || t->dim != 1 || t->strides[0] != 1) return false;
  a->size           = t->sizes[0];
  a->storage_offset = t->storage_offset;
  a->dtype          = t->dtype;
  return true;
}

bool wholegraph_convert_tensor_desc_to_matrix(wholegraph_matrix_description_t* m,
                                               wholegraph_tensor_description_t* t)
{
  if (!known_dtype(t->dtype)) return false;
  if (t->dim != 1 && t->dim != 2) return false;
  if (t->dim == 2 && t->strides[1] != 1) return false;
  m->dtype          = t->dtype;
  m->storage_offset = t->storage_offset;
  m->sizes[0]       = t->sizes[0];
  m->sizes[1]       = t->dim == 2 ? t->sizes[1] : 1;
  m->stride         = t->dim == 2 ? t->strides[0] : 1;
  return true;
}

int64_t wholegraph_get_memory_element_count_from_array(wholegraph_array_description_t* a)
{
  return a->size;
}
int64_t wholegraph_get_memory_size_from_array(wholegraph_array_description_t* a)
{
  return a->size * static_cast<int64_t>(wholegraph_dtype_get_element_size(a->dtype));
}
int64_t wholegraph_get_memory_element_count_from_matrix(wholegraph_matrix_description_t* m)
{
  return m->sizes[0] * m->stride;
}
int64_t wholegraph_get_memory_size_from_matrix(wholegraph_matrix_description_t* m)
{
  return m->sizes[0] * m->stride * static_cast<int64_t>(wholegraph_dtype_get_element_size(m->dtype));
}
int64_t wholegraph_get_memory_element_count_from_tensor(wholegraph_tensor_description_t* t)
{
  if (t->dim == 0) return 1;
  if (t->dim < 0 || t->dim >= WHOLEGRAPH_MAX_TENSOR_DIM) return -1;
  return t->strides[0] * t->sizes[0];
}
int64_t wholegraph_get_memory_size_from_tensor(wholegraph_tensor_description_t* t)
{
  return wholegraph_get_memory_element_count_from_tensor(t) *
         static_cast<int64_t>(wholegraph_dtype_get_element_size(t->dtype));
}

bool wholegraph_squeeze_tensor(wholegraph_tensor_description_t* t, int dim)
{
  if (t == nullptr || dim < 0 || dim >= t->dim || t->sizes[dim] != 1) return false;
  if (dim != t->dim - 1 && t->strides[dim] != t->strides[dim + 1]) return false;
  for (int i = dim; i + 1 < t->dim; i++) {
    t->sizes[i]   = t->sizes[i + 1];
    t->strides[i] = t->strides[i + 1];
  }
  t->dim--;
  return true;
}

bool wholegraph_unsqueeze_tensor(wholegraph_tensor_description_t* t, int dim)
{
  if (t == nullptr || dim < 0 || dim > t->dim || t->dim + 1 > WHOLEGRAPH_MAX_TENSOR_DIM)
    return false;
  // The new axis takes the stride of the axis it displaces (or of the last axis when appended).
  int64_t stride = t->dim > 0 ? t->strides[t->dim - 1] : 1;
  for (int i = t->dim; i > dim; i--) {
    t->sizes[i]   = t->sizes[i - 1];
    t->strides[i] = t->strides[i - 1];
    stride        = t->strides[i];
  }
  t->sizes[dim]   = 1;
  t->strides[dim] = stride;
  t->dim++;
  return true;
}

wholegraph_gref_t wholegraph_create_continuous_global_reference(void* ptr)
{
  wholegraph_gref_t g;
  g.pointer = ptr;
  return g;
}

}  // extern "C"
