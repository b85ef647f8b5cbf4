/*
 * wholegraph-b200: dtype enum and array / matrix / tensor descriptors.
 *
 * ABI mirror of the reference's cpp/include/wholegraph/tensor_description.h
 * (enum values :18-29, struct layouts :56-88, helpers :97-226). All sizes,
 * strides and storage offsets count ELEMENTS, never bytes.
 */
#pragma once

#include <stdint.h>
#include <stdlib.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Element types. Values are part of the ABI (tensor_description.h:18-29). */
enum wholegraph_dtype_t {
  WHOLEGRAPH_DT_UNKNOWN = 0,
  WHOLEGRAPH_DT_FLOAT,  /* 1: fp32 */
  WHOLEGRAPH_DT_HALF,   /* 2: fp16 */
  WHOLEGRAPH_DT_DOUBLE, /* 3: fp64 */
  WHOLEGRAPH_DT_BF16,   /* 4: bfloat16 */
  WHOLEGRAPH_DT_INT,    /* 5: int32 */
  WHOLEGRAPH_DT_INT64,  /* 6: int64 */
  WHOLEGRAPH_DT_INT16,  /* 7: int16 */
  WHOLEGRAPH_DT_INT8,   /* 8: int8 */
  WHOLEGRAPH_DT_COUNT,  /* 9: number of values */
};

/* Bytes per element; 0 for UNKNOWN, (size_t)-1 for an out-of-range value. */
size_t wholegraph_dtype_get_element_size(wholegraph_dtype_t dtype);
bool wholegraph_dtype_is_floating_number(wholegraph_dtype_t dtype);
bool wholegraph_dtype_is_integer_number(wholegraph_dtype_t dtype);

/* 1-D view. */
struct wholegraph_array_description_t {
  int64_t size;
  int64_t storage_offset;
  wholegraph_dtype_t dtype;
};

/* 2-D row-major view; `stride` is the distance between rows. */
struct wholegraph_matrix_description_t {
  int64_t sizes[2];
  int64_t stride;
  int64_t storage_offset;
  wholegraph_dtype_t dtype;
};

#define WHOLEGRAPH_MAX_TENSOR_DIM (8)

/* N-D view (N <= 8). */
struct wholegraph_tensor_description_t {
  int64_t sizes[WHOLEGRAPH_MAX_TENSOR_DIM];
  int64_t strides[WHOLEGRAPH_MAX_TENSOR_DIM];
  int64_t storage_offset;
  int dim;
  wholegraph_dtype_t dtype;
};

wholegraph_array_description_t wholegraph_create_array_desc(int64_t size,
                                                              int64_t storage_offset,
                                                              wholegraph_dtype_t dtype);

wholegraph_matrix_description_t wholegraph_create_matrix_desc(int64_t sizes[2],
                                                                int64_t stride,
                                                                int64_t storage_offset,
                                                                wholegraph_dtype_t dtype);

/* dim = 0, every size and stride 1, offset 0, dtype UNKNOWN. */
void wholegraph_initialize_tensor_desc(wholegraph_tensor_description_t* p_tensor_description);

void wholegraph_copy_array_desc_to_matrix(wholegraph_matrix_description_t* p_matrix_description,
                                           wholegraph_array_description_t* p_array_description);
void wholegraph_copy_array_desc_to_tensor(wholegraph_tensor_description_t* p_tensor_description,
                                           wholegraph_array_description_t* p_array_description);
void wholegraph_copy_matrix_desc_to_tensor(wholegraph_tensor_description_t* p_tensor_description,
                                            wholegraph_matrix_description_t* p_matrix_description);

/* False unless the tensor is 1-D with unit stride and a known dtype. */
bool wholegraph_convert_tensor_desc_to_array(
  wholegraph_array_description_t* p_array_description,
  wholegraph_tensor_description_t* p_tensor_description);

/* False unless the tensor is 1-D, or 2-D with a unit inner stride, and has a known dtype. */
bool wholegraph_convert_tensor_desc_to_matrix(
  wholegraph_matrix_description_t* p_matrix_description,
  wholegraph_tensor_description_t* p_tensor_description);

int64_t wholegraph_get_memory_element_count_from_array(
  wholegraph_array_description_t* p_array_description);
int64_t wholegraph_get_memory_size_from_array(
  wholegraph_array_description_t* p_array_description);
int64_t wholegraph_get_memory_element_count_from_matrix(
  wholegraph_matrix_description_t* p_matrix_description);
int64_t wholegraph_get_memory_size_from_matrix(
  wholegraph_matrix_description_t* p_matrix_description);
int64_t wholegraph_get_memory_element_count_from_tensor(
  wholegraph_tensor_description_t* p_tensor_description);
int64_t wholegraph_get_memory_size_from_tensor(
  wholegraph_tensor_description_t* p_tensor_description);

/* Drop / insert a size-1 dimension in place; false when not possible. */
bool wholegraph_squeeze_tensor(wholegraph_tensor_description_t* p_tensor_description, int dim);
bool wholegraph_unsqueeze_tensor(wholegraph_tensor_description_t* p_tensor_description, int dim);

#ifdef __cplusplus
}
#endif
