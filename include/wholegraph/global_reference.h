/*
 * wholegraph-b200: global reference to a mapped table.
 *
 * ABI mirror of the reference's cpp/include/wholegraph/global_reference.h:19-29.
 * A global reference is a bare pointer to the first byte of a table that every
 * rank can dereference (one rank's buffer, or the single virtual range into
 * which all ranks' shards of a CONTINUOUS allocation are mapped).
 */
#pragma once

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

struct wholegraph_gref_t {
  void* pointer; /* first byte of the mapped data */
};

/* Wrap a plain pointer as a global reference (global_reference.h:29). */
wholegraph_gref_t wholegraph_create_continuous_global_reference(void* ptr);

#ifdef __cplusplus
}
#endif
