// CPU runtime, part 2: host-side allocators that hand out *indices/offsets* into device pools.
//
//  * BlockAllocator: fixed-size KV-cache pages with a LIFO free list and per-sequence block lists
//    (the reference's paged cache keeps a block table per sequence and grows it page by page:
//    scirust-core/src/nn/paged_attention.rs:21-147). Freed pages are reused most-recent-first so
//    a workload's physical layout is reproducible.
//  * Arena: a bump allocator over one preallocated device buffer with mark/release, used for the
//    step-scoped workspace instead of one allocation per op (the reference's op-chain allocates an
//    output for every op: scirust-cuda/src/chain.rs:1049-1052; its CPU arenas:
//    scirust-arena/src/*).
#include <stdint.h>
#include <stdlib.h>

#include <vector>

struct SbBlockAlloc {
  std::vector<int32_t> free_list;
  int32_t n_blocks;
};
struct SbArena {
  uint64_t capacity, offset, high_water;
};

extern "C" {

SbBlockAlloc* sbrt_balloc_new(int32_t n_blocks) {
  if (n_blocks <= 0) return nullptr;
  SbBlockAlloc* a = new SbBlockAlloc();
  a->n_blocks = n_blocks;
  a->free_list.reserve(n_blocks);
  for (int32_t i = n_blocks - 1; i >= 0; --i) a->free_list.push_back(i);  // block 0 is handed out first
  return a;
}
void sbrt_balloc_delete(SbBlockAlloc* a) { delete a; }
int32_t sbrt_balloc_num_free(const SbBlockAlloc* a) { return static_cast<int32_t>(a->free_list.size()); }
// Allocates n blocks into out[]; returns 0, or -1 (and allocates nothing) if fewer than n are free.
int32_t sbrt_balloc_alloc(SbBlockAlloc* a, int32_t n, int32_t* out) {
  if (n < 0 || static_cast<size_t>(n) > a->free_list.size()) return -1;
  for (int32_t i = 0; i < n; ++i) {
    out[i] = a->free_list.back();
    a->free_list.pop_back();
  }
  return 0;
}
// Returns blocks to the pool; ids outside the pool are rejected (-1) and nothing is freed.
int32_t sbrt_balloc_free(SbBlockAlloc* a, const int32_t* ids, int32_t n) {
  for (int32_t i = 0; i < n; ++i)
    if (ids[i] < 0 || ids[i] >= a->n_blocks) return -1;
  if (a->free_list.size() + static_cast<size_t>(n) > static_cast<size_t>(a->n_blocks)) return -1;
  for (int32_t i = 0; i < n; ++i) a->free_list.push_back(ids[i]);
  return 0;
}

SbArena* sbrt_arena_new(uint64_t capacity) {
  SbArena* a = new SbArena();
  a->capacity = capacity;
  a->offset = 0;
  a->high_water = 0;
  return a;
}
void sbrt_arena_delete(SbArena* a) { delete a; }
// Returns the byte offset of an `align`-aligned block of `bytes`, or UINT64_MAX when exhausted.
uint64_t sbrt_arena_alloc(SbArena* a, uint64_t bytes, uint64_t align) {
  if (align == 0) align = 256;
  const uint64_t start = (a->offset + align - 1) / align * align;
  if (start + bytes > a->capacity) return UINT64_MAX;
  a->offset = start + bytes;
  if (a->offset > a->high_water) a->high_water = a->offset;
  return start;
}
uint64_t sbrt_arena_mark(const SbArena* a) { return a->offset; }
void sbrt_arena_release(SbArena* a, uint64_t mark) {
  if (mark <= a->offset) a->offset = mark;
}
uint64_t sbrt_arena_high_water(const SbArena* a) { return a->high_water; }

}  // extern "C"
