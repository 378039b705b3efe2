// CPU check of include/b200q.hpp: every case must be rejected on the host (std::invalid_argument)
// before any CUDA call, with the reference's wording.  Prints SHIM-OK on success.
#include <cstdio>
#include <cstring>

#include "b200q.hpp"

using namespace b200q;

static ArrayView view(Dtype t, std::vector<int64_t> shape) {
  ArrayView a;
  a.data = reinterpret_cast<void*>(0x1000);
  a.dtype = t;
  a.shape = std::move(shape);
  return a;
}
template <class F>
static int expect_invalid(const char* what, const char* needle, F f) {
  try {
    f();
  } catch (const std::invalid_argument& e) {
    if (std::strstr(e.what(), needle)) return 0;
    std::printf("%s: wrong message: %s\n", what, e.what());
    return 1;
  } catch (const std::exception& e) {
    std::printf("%s: wrong exception: %s\n", what, e.what());
    return 1;
  }
  std::printf("%s: not rejected\n", what);
  return 1;
}

int main() {
  int bad = 0;
  Workspace ws{reinterpret_cast<void*>(0x2000), 1 << 20};
  auto x = view(Dtype::bfloat16, {4, 512});
  auto w = view(Dtype::uint32, {256, 64});       // 4-bit: K = 512
  auto s = view(Dtype::bfloat16, {256, 8});
  auto b = view(Dtype::bfloat16, {256, 8});
  auto out = view(Dtype::bfloat16, {4, 256});
  bad += expect_invalid("float weights", "should be uint32", [&] {
    auto wf = view(Dtype::float32, {256, 64});
    quantized_matmul(x, wf, s, b, out, ws);
  });
  bad += expect_invalid("scales/biases shapes", "Scales and biases should have the same shape", [&] {
    auto b2 = view(Dtype::bfloat16, {256, 4});
    quantized_matmul(x, w, s, b2, out, ws);
  });
  bad += expect_invalid("batch shape", "same batch shape", [&] {
    auto s3 = view(Dtype::bfloat16, {2, 256, 8});
    auto b3 = view(Dtype::bfloat16, {2, 256, 8});
    quantized_matmul(x, w, s3, b3, out, ws);
  });
  bad += expect_invalid("bits vs shapes", "incompatible based on bits and group_size", [&] { quantized_matmul(x, w, s, b, out, ws, true, 64, 8); });
  bad += expect_invalid("inner dimension", "does not match the expanded quantized matrix", [&] {
    auto x2 = view(Dtype::bfloat16, {4, 256});
    quantized_matmul(x2, w, s, b, out, ws);
  });
  bad += expect_invalid("group size", "The requested group size 48 is not supported", [&] {
    auto s48 = view(Dtype::bfloat16, {256, 512 / 48 + 1});
    (void)s48;
    auto wq = view(Dtype::uint32, {8, 6});
    auto sc = view(Dtype::float32, {8, 1});
    auto bi = view(Dtype::float32, {8, 1});
    auto wf = view(Dtype::float32, {8, 48});
    quantize(wf, wq, sc, bi, 48, 4);
  });
  bad += expect_invalid("quantize integer input", "Only real floating types can be quantized", [&] {
    auto wi = view(Dtype::uint32, {8, 64});
    quantize(wi, w, s, b);
  });
  bad += expect_invalid("quantize 1-D", "at least 2 dimension", [&] {
    auto w1 = view(Dtype::float32, {64});
    quantize(w1, w, s, b);
  });
  bad += expect_invalid("embedding ids dtype", "ids must be uint32", [&] {
    auto ids = view(Dtype::float32, {5});
    auto eo = view(Dtype::bfloat16, {5, 512});
    quantized_embedding(ids, w, s, b, eo);
  });
  bad += expect_invalid("embedding table shapes", "Scales and biases should have the same shape", [&] {
    auto ids = view(Dtype::uint32, {5});
    auto b2 = view(Dtype::bfloat16, {256, 4});
    auto eo = view(Dtype::bfloat16, {5, 512});
    quantized_embedding(ids, w, s, b2, eo);
  });
  bad += expect_invalid("gather index dtype", "Indices must be integral", [&] {
    auto xe = view(Dtype::bfloat16, {4, 1, 512});
    auto we = view(Dtype::uint32, {2, 256, 64});
    auto se = view(Dtype::bfloat16, {2, 256, 8});
    auto li = view(Dtype::float32, {4});
    auto ri = view(Dtype::uint32, {4});
    gather_qmm(xe, we, se, se, li, ri, out, ws);
  });
  if (bad == 0) std::printf("SHIM-OK\n");
  return bad;
}
