// TEST INFRASTRUCTURE ONLY. Runs the reference's own C++ host oracle on inputs from a file and writes its answers, so
// that golden vectors of it can be committed (tests/golden/make_golden.py) and oracle/decode_gemv_oracle.py checked
// against an implementation that shares no code with torch.
//
// The reference headers are included from where they lie in the reference checkout (-I .../fp8-block-rows/tests/order):
//   row_fp8.h    crit::fp8::decode (:25-31, E4M3 byte -> float), crit::fp8::project (:86-98, FP64 projection of FP8
//                codes with BF16 row scales)
//   fp8_block.h  crit::fp8_block::e8m0 (:18-21), quantize_group (:24-39, the MX shared exponent
//                2^(floor(log2 amax) - 8) and the E4M3 codes of a 32-group)
//
// Input file (little endian): int32 rows, width, tokens, groups; codes u8[rows*width] (no NaN codes);
// scales u16[rows] (BF16 words, non-negative); x u16[tokens*width] (BF16 words); values f32[groups*32].
// Output file: decode f32[256] (NaN for the two NaN codes); project f64[tokens*rows];
// per group: scale f32, e8m0 check f32 (e8m0(byte of that scale)), codes u8[32].
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <limits>
#include <vector>

#include "fp8_block.h"

namespace {

template <typename T>
bool read(std::FILE* f, std::vector<T>& v) {
  return v.empty() || std::fread(v.data(), sizeof(T), v.size(), f) == v.size();
}
template <typename T>
bool write(std::FILE* f, const std::vector<T>& v) {
  return v.empty() || std::fwrite(v.data(), sizeof(T), v.size(), f) == v.size();
}

}  // namespace

int main(int argc, char** argv) {
  if (argc != 3) {
    std::fprintf(stderr, "usage: %s input output\n", argv[0]);
    return 2;
  }
  std::FILE* in = std::fopen(argv[1], "rb");
  if (!in) return 3;
  std::int32_t head[4];
  if (std::fread(head, sizeof(std::int32_t), 4, in) != 4) return 3;
  const std::size_t rows = head[0], width = head[1], tokens = head[2], groups = head[3];
  crit::fp8::RowWeights w{rows, width, std::vector<std::uint8_t>(rows * width), std::vector<std::uint16_t>(rows)};
  std::vector<std::uint16_t> x(tokens * width);
  std::vector<float> values(groups * 32);
  if (!read(in, w.codes) || !read(in, w.scales) || !read(in, x) || !read(in, values)) return 3;
  std::fclose(in);

  std::vector<float> table(256);
  for (int code = 0; code < 256; ++code)
    table[code] = (code & 127) == 127 ? std::numeric_limits<float>::quiet_NaN()
                                      : crit::fp8::decode(static_cast<std::uint8_t>(code));
  const std::vector<double> projected = crit::fp8::project(w, x, tokens);

  std::FILE* out = std::fopen(argv[2], "wb");
  if (!out || !write(out, table) || !write(out, projected)) return 4;
  for (std::size_t g = 0; g < groups; ++g) {
    std::vector<std::uint8_t> codes(32);
    const float scale =
        crit::fp8_block::quantize_group(values.data() + 32 * g, 32, crit::fp8_block::ScaleKind::mx, codes.data());
    int e = 0;
    (void)std::frexp(scale, &e);   // scale = 2^(e - 1): its E8M0 byte is e - 1 + 127
    const float back = crit::fp8_block::e8m0(static_cast<std::uint8_t>(e - 1 + 127));
    const std::vector<float> pair = {scale, back};
    if (!write(out, pair) || !write(out, codes)) return 4;
  }
  std::fclose(out);
  return 0;
}
