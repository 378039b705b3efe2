// TEST INFRASTRUCTURE ONLY - never linked into, imported by or executed from the product
// library.  Compiles the reference project's GGUF repack translation unit from the reference
// checkout (nothing of it is copied here; the third-party header it needs is replaced by the
// declarations in oracle/stub/gguflib.h) and drives the one function of it that is pure:
//   unpack_32_4   mlx/io/gguf_quants.cpp:13-31   (32 four-bit weights of a block -> 16 bytes in
//                                                 the affine layout's nibble order)
// The extract_* loops around it take the reference's array objects, whose runtime is not
// linked; they are restated in gguf_ref.c.
//
// Usage: ref_gguf unpack <n_blocks> in.bin out.bin     (16 bytes in, 16 bytes out per block)
#include "mlx/io/gguf_quants.cpp"

#include <cstdio>
#include <cstdlib>
#include <vector>

int main(int argc, char** argv) {
  if (argc != 5 || std::string(argv[1]) != "unpack") {
    std::fprintf(stderr, "usage: ref_gguf unpack <n_blocks> in.bin out.bin\n");
    return 2;
  }
  const size_t n = std::strtoull(argv[2], nullptr, 10);
  std::vector<uint8_t> in(16 * n), out(16 * n);
  FILE* f = std::fopen(argv[3], "rb");
  if (!f || std::fread(in.data(), 1, in.size(), f) != in.size()) return 2;
  std::fclose(f);
  for (size_t i = 0; i < n; ++i)
    mlx::core::unpack_32_4(in.data() + 16 * i, reinterpret_cast<int8_t*>(out.data() + 16 * i));
  f = std::fopen(argv[4], "wb");
  if (!f || std::fwrite(out.data(), 1, out.size(), f) != out.size()) return 2;
  std::fclose(f);
  return 0;
}
