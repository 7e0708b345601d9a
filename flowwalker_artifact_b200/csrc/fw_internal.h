// Internal definitions shared by the translation units of libflowwalker.
#pragma once
#include <stdarg.h>
#include <stdint.h>
#include <stdlib.h>

#include "../../include/flowwalker.h"

// Host CSR.  Arrays are malloc'ed; xadj holds V+1 offsets of xadj_bits each.
struct fw_graph {
  int64_t V = 0;
  int64_t E = 0;
  int32_t xadj_bits = 32;
  void* xadj = nullptr;
  int32_t* adj = nullptr;
  float* weight = nullptr;
  int32_t* label = nullptr;
};

namespace fw {
// Records the message returned by fw_last_error() and passes `code` through.
int fail(int code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));
void clear_error();

inline int64_t row_begin(const fw_graph* g, int64_t v) {
  return g->xadj_bits == 64 ? static_cast<const int64_t*>(g->xadj)[v]
                            : (int64_t) static_cast<const uint32_t*>(g->xadj)[v];
}
}  // namespace fw
