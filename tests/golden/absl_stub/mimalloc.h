// A stand-in for the two mimalloc calls the reference's host allocator makes, on the C
// library, so that the file compiles on a machine without mimalloc.
#pragma once
#include <cstddef>
#include <cstdlib>

inline void* mi_malloc_aligned(size_t bytes, size_t alignment) {
  if (alignment < sizeof(void*)) alignment = sizeof(void*);
  const size_t rounded = (bytes + alignment - 1) / alignment * alignment;
  return std::aligned_alloc(alignment, rounded ? rounded : alignment);
}
inline void mi_free(void* p) { std::free(p); }
