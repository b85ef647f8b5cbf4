// wholegraph_load_from_file / wholegraph_store_to_file: raw row-major records, one record per
// table row, optionally narrower in the file than in memory.
// Behaviour follows the reference's cpp/src/wholegraph/file_io.cpp (load :1849-2046, store
// :2048-2165): plain layout and round-robin blocks; buffered reads only (no O_DIRECT variant).
#include <sys/stat.h>

#include <algorithm>
#include <cstdio>
#include <string>
#include <vector>

#include <wholegraph/wholegraph.h>

#include "common.hpp"
#include "handle.hpp"

namespace {

// Sequential reader over the logical concatenation of several files of fixed-size records.
class record_reader {
 public:
  record_reader(const char** names, const std::vector<size_t>& entries, size_t record_bytes)
    : names_(names), entries_(entries), record_bytes_(record_bytes)
  {
  }
  ~record_reader()
  {
    if (fp_) fclose(fp_);
  }
  // Records [first, first + count) -> dst, `dst_stride` bytes apart.
  void read(size_t first, size_t count, char* dst, size_t dst_stride)
  {
    for (size_t i = 0; i < count; i++) {
      const size_t r = first + i;
      if (fp_ == nullptr || r < file_first_ || r >= file_first_ + entries_[file_] || r != next_) seek(r);
      if (fread(dst + i * dst_stride, 1, record_bytes_, fp_) != record_bytes_)
        throw wgb::system_error(std::string("short read from ") + names_[file_]);
      next_ = r + 1;
    }
  }

 private:
  void seek(size_t r)
  {
    size_t f = 0, start = 0;
    while (f < entries_.size() && start + entries_[f] <= r) start += entries_[f++];
    if (f == entries_.size()) throw wgb::logic_error("record past the end of the files");
    if (fp_ == nullptr || f != file_) {
      if (fp_) fclose(fp_);
      fp_ = fopen(names_[f], "rb");
      if (fp_ == nullptr) throw wgb::system_error(std::string("cannot open ") + names_[f]);
    }
    file_ = f, file_first_ = start;
    if (fseeko(fp_, static_cast<off_t>((r - start) * record_bytes_), SEEK_SET) != 0)
      throw wgb::system_error(std::string("cannot seek in ") + names_[f]);
  }
  const char** names_;
  const std::vector<size_t>& entries_;
  size_t record_bytes_;
  FILE* fp_         = nullptr;
  size_t file_      = 0;
  size_t file_first_ = 0;
  size_t next_      = static_cast<size_t>(-1);
};

}  // namespace

extern "C" {

wholegraph_error_code_t wholegraph_load_from_file(wholegraph_handle_t h,
                                                    size_t memory_offset,
                                                    size_t memory_entry_size,
                                                    size_t file_entry_size,
                                                    const char** file_names,
                                                    int file_count,
                                                    int round_robin_size)
{
  if (h == nullptr || file_names == nullptr || file_count <= 0 || file_count >= 65536) return WHOLEGRAPH_INVALID_INPUT;
  if (file_entry_size == 0 || memory_entry_size < file_entry_size) return WHOLEGRAPH_INVALID_INPUT;
  if (round_robin_size < 0) return WHOLEGRAPH_INVALID_INPUT;
  WGB_API_BEGIN
  std::vector<size_t> file_entries(file_count);
  size_t total_entries = 0;
  for (int f = 0; f < file_count; f++) {
    if (file_names[f] == nullptr) throw wgb::invalid_input(WHOLEGRAPH_INVALID_INPUT, "a file name is null");
    struct stat st;
    if (stat(file_names[f], &st) != 0)
      throw wgb::invalid_input(WHOLEGRAPH_INVALID_INPUT, std::string("cannot stat ") + file_names[f]);
    if (static_cast<size_t>(st.st_size) % file_entry_size != 0)
      throw wgb::invalid_input(WHOLEGRAPH_INVALID_INPUT, std::string(file_names[f]) + " holds a partial record");
    file_entries[f] = static_cast<size_t>(st.st_size) / file_entry_size;
    total_entries += file_entries[f];
  }
  if (!h->comm->all_same(file_entries.data(), sizeof(size_t) * file_count))
    throw wgb::comm_error("the ranks see files of different sizes");
  const int me    = h->comm->world_rank;
  const int W     = h->comm->world_size;
  const size_t lo = h->part_offsets[me];
  const size_t hi = lo + h->part_sizes[me];
  record_reader reader(file_names, file_entries, file_entry_size);
  const size_t batch = std::max<size_t>(1, (size_t(64) << 20) / memory_entry_size);
  std::vector<char> staging(batch * memory_entry_size, 0);
  // `count` consecutive records from `first` -> consecutive slots of this rank's shard from byte `at`.
  auto place = [&](size_t first, size_t count, size_t at) {
    for (size_t done = 0; done < count; done += batch) {
      const size_t now = std::min(batch, count - done);
      reader.read(first + done, now, staging.data(), memory_entry_size);
      char* dst = static_cast<char*>(h->local_ptr) + at + done * memory_entry_size;
      WGB_CUDA_CHECK(cudaMemcpy2D(dst, memory_entry_size, staging.data(), memory_entry_size, file_entry_size, now,
                                  cudaMemcpyDefault));
    }
  };
  if (round_robin_size == 0) {
    // Record r of the logical concatenation of the files lands at memory_offset + r * memory_entry_size;
    // each rank loads the records whose slot starts inside its own shard.
    if (memory_offset + total_entries * memory_entry_size > h->total_size + (memory_entry_size - file_entry_size))
      throw wgb::invalid_input(WHOLEGRAPH_INVALID_VALUE, "the files hold more records than the allocation");
    size_t first = lo <= memory_offset ? 0 : (lo - memory_offset + memory_entry_size - 1) / memory_entry_size;
    size_t last  = hi <= memory_offset ? 0 : (hi - memory_offset + memory_entry_size - 1) / memory_entry_size;
    if (last > total_entries) last = total_entries;
    if (first < last) place(first, last - first, memory_offset + first * memory_entry_size - lo);
  } else {
    // Blocks of round_robin_size records are dealt to the ranks in turn: block b goes to rank b % W
    // and is that rank's block b / W (reference: file_io.cpp:100-200).  The memory offset can only
    // name a column inside the slot here.
    const size_t rr = static_cast<size_t>(round_robin_size);
    if (memory_offset + file_entry_size > memory_entry_size)
      throw wgb::invalid_input(WHOLEGRAPH_INVALID_INPUT, "with round robin the memory offset must stay inside a slot");
    if (rr > total_entries / W) throw wgb::invalid_input(WHOLEGRAPH_INVALID_VALUE, "illegal round_robin_size");
    const size_t extra = total_entries % (W * rr);
    size_t local_count = total_entries / (W * rr) * rr;
    if (extra > static_cast<size_t>(me) * rr) local_count += std::min(rr, extra - static_cast<size_t>(me) * rr);
    if (memory_offset + (local_count == 0 ? 0 : (local_count - 1) * memory_entry_size + file_entry_size) > hi - lo)
      throw wgb::invalid_input(WHOLEGRAPH_INVALID_VALUE, "this rank's records do not fit its shard");
    for (size_t done = 0; done < local_count; done += rr) {
      const size_t now   = std::min(rr, local_count - done);
      const size_t block = done / rr;
      place((block * W + me) * rr, now, memory_offset + done * memory_entry_size);
    }
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
