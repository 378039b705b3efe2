/* TEST INFRASTRUCTURE ONLY.  Stand-in for the third-party gguflib header that the reference's
 * build fetches from the network (antirez/gguf-tools): just enough declarations for
 * mlx/io/gguf_quants.cpp to compile, so that its pure nibble re-ordering function can be run as
 * a checker.  Written from the published GGUF type numbering; no code of that library is here. */
#ifndef B200Q_ORACLE_GGUFLIB_STUB_H
#define B200Q_ORACLE_GGUFLIB_STUB_H
#include <stddef.h>
#include <stdint.h>
enum { GGUF_TYPE_F32 = 0, GGUF_TYPE_F16 = 1, GGUF_TYPE_Q4_0 = 2, GGUF_TYPE_Q4_1 = 3, GGUF_TYPE_Q8_0 = 8 };
#define GGUF_TENSOR_MAX_DIM 8
typedef struct {
  const char* name;
  size_t namelen;
  uint32_t type;
  uint32_t ndim;
  uint64_t dim[GGUF_TENSOR_MAX_DIM];
  uint64_t offset;
  uint64_t bsize;
  uint64_t num_weights;
  uint8_t* weights_data;
} gguf_tensor;
#endif
