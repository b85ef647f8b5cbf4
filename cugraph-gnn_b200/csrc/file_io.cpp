// wholegraph_load_from_file / wholegraph_store_to_file: raw row-major records, one record per
// table row, optionally narrower in the file than in memory.
// Behaviour follows the reference's cpp/src/wholegraph/file_io.cpp (load :1849-2046, store
// :2048-2165) for the plain layout; the round-robin layout is not implemented.
#include <sys/stat.h>

#include <cstdio>
#include <vector>

#include <wholegraph/wholegraph.h>

#include "common.hpp"
#include "handle.hpp"

extern "C" {

wholegraph_error_code_t wholegraph_load_from_file(wholegraph_handle_t h,
                                                    size_t memory_offset,
                                                    size_t memory_entry_size,
                                                    size_t file_entry_size,
                                                    const char** file_names,
                                                    int file_count,
                                                    int round_robin_size)
{
  if (h == nullptr || file_names == nullptr || file_count <= 0) return WHOLEGRAPH_INVALID_INPUT;
  if (file_entry_size == 0 || memory_entry_size < file_entry_size) return WHOLEGRAPH_INVALID_VALUE;
  if (round_robin_size != 0) return WHOLEGRAPH_NOT_IMPLEMENTED;
  WGB_API_BEGIN
  // Record r of the logical concatenation of the files lands at
  // memory_offset + r * memory_entry_size; each rank loads the records of its own shard.
  std::vector<size_t> file_entries(file_count);
  size_t total_entries = 0;
  for (int f = 0; f < file_count; f++) {
    struct stat st;
    if (stat(file_names[f], &st) != 0)
      throw wgb::system_error(std::string("cannot stat ") + file_names[f]);
    if (static_cast<size_t>(st.st_size) % file_entry_size != 0)
      throw wgb::invalid_input(WHOLEGRAPH_INVALID_VALUE, std::string(file_names[f]) + " holds a partial record");
    file_entries[f] = static_cast<size_t>(st.st_size) / file_entry_size;
    total_entries += file_entries[f];
  }
  if (memory_offset + total_entries * memory_entry_size > h->total_size + (memory_entry_size - file_entry_size))
    throw wgb::invalid_input(WHOLEGRAPH_INVALID_VALUE, "the files hold more records than the allocation");
  const int me          = h->comm->world_rank;
  const size_t lo       = h->part_offsets[me];
  const size_t hi       = lo + h->part_sizes[me];
  // first / last record whose memory slot starts inside this rank's shard
  size_t first = lo <= memory_offset ? 0 : (lo - memory_offset + memory_entry_size - 1) / memory_entry_size;
  size_t last  = hi <= memory_offset ? 0 : (hi - memory_offset + memory_entry_size - 1) / memory_entry_size;
  if (last > total_entries) last = total_entries;
  if (first < last) {
    const size_t batch = std::max<size_t>(1, (size_t(64) << 20) / memory_entry_size);
    std::vector<char> staging(batch * memory_entry_size, 0);
    size_t rec = first, file = 0, file_first = 0;
    while (file < static_cast<size_t>(file_count) && file_first + file_entries[file] <= rec)
      file_first += file_entries[file++];
    FILE* fp = nullptr;
    while (rec < last) {
      const size_t now = std::min(batch, last - rec);
      for (size_t i = 0; i < now; i++) {
        const size_t r = rec + i;
        while (file_first + file_entries[file] <= r) {
          file_first += file_entries[file++];
          if (fp) fclose(fp), fp = nullptr;
        }
        if (fp == nullptr) {
          fp = fopen(file_names[file], "rb");
          if (fp == nullptr) throw wgb::system_error(std::string("cannot open ") + file_names[file]);
          fseeko(fp, static_cast<off_t>((r - file_first) * file_entry_size), SEEK_SET);
        }
        if (fread(staging.data() + i * memory_entry_size, 1, file_entry_size, fp) != file_entry_size) {
          fclose(fp);
          throw wgb::system_error(std::string("short read from ") + file_names[file]);
        }
      }
      char* dst = static_cast<char*>(h->local_ptr) + (memory_offset + rec * memory_entry_size - lo);
      WGB_CUDA_CHECK(cudaMemcpy2D(dst, memory_entry_size, staging.data(), memory_entry_size, file_entry_size,
                                  now, cudaMemcpyDefault));
      rec += now;
    }
    if (fp) fclose(fp);
  }
  h->comm->barrier();
  return WHOLEGRAPH_SUCCESS;
  WGB_API_END("wholegraph_load_from_file")
}

wholegraph_error_code_t wholegraph_store_to_file(wholegraph_handle_t h,
                                                   size_t memory_offset,
                                                   size_t memory_entry_stride,
                                                   size_t file_entry_size,
                                                   const char* local_file_name)
{
  if (h == nullptr || local_file_name == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  if (file_entry_size == 0 || memory_entry_stride < file_entry_size) return WHOLEGRAPH_INVALID_VALUE;
  WGB_API_BEGIN
  const int me    = h->comm->world_rank;
  const size_t lo = h->part_offsets[me];
  const size_t hi = lo + h->part_sizes[me];
  size_t first = lo <= memory_offset ? 0 : (lo - memory_offset + memory_entry_stride - 1) / memory_entry_stride;
  size_t last  = hi <= memory_offset ? 0 : (hi - memory_offset + memory_entry_stride - 1) / memory_entry_stride;
  FILE* fp     = fopen(local_file_name, "wb");
  if (fp == nullptr) throw wgb::system_error(std::string("cannot create ") + local_file_name);
  const size_t batch = std::max<size_t>(1, (size_t(64) << 20) / file_entry_size);
  std::vector<char> staging(batch * file_entry_size);
  for (size_t rec = first; rec < last; rec += batch) {
    const size_t now = std::min(batch, last - rec);
    const char* src  = static_cast<const char*>(h->local_ptr) + (memory_offset + rec * memory_entry_stride - lo);
    cudaError_t e    = cudaMemcpy2D(staging.data(), file_entry_size, src, memory_entry_stride, file_entry_size,
                                    now, cudaMemcpyDefault);
    if (e != cudaSuccess || fwrite(staging.data(), file_entry_size, now, fp) != now) {
      fclose(fp);
      throw wgb::system_error(std::string("cannot write ") + local_file_name);
    }
  }
  fclose(fp);
  h->comm->barrier();
  return WHOLEGRAPH_SUCCESS;
  WGB_API_END("wholegraph_store_to_file")
}

}  // extern "C"
