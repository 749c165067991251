// DecodePfm: host-side parser of an in-memory PFM file (reference: custom_helper_op/cc/kernels/
// pfm_decoder_kernels.cc:38-116, a CPU OpKernel).  Follows the reference statement by statement, including its
// treatment of a comment line (skipped up to, not past, its newline, after which the width fails to parse).
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>

#include "../../include/chop.h"

namespace {

const char* const kWs = " \t\r\n";

int fail(char* msg, size_t cap, const std::string& text) {
  if (msg && cap) {
    std::snprintf(msg, cap, "%s", text.c_str());
  }
  return CHOP_ERR_FORMAT;
}

bool parse_i64(const std::string& s, int64_t* v) {
  if (s.empty()) return false;
  char* end = nullptr;
  const long long x = std::strtoll(s.c_str(), &end, 10);
  if (end != s.c_str() + s.size()) return false;
  *v = x;
  return true;
}

bool parse_f32(const std::string& s, float* v) {
  if (s.empty()) return false;
  char* end = nullptr;
  const float x = std::strtof(s.c_str(), &end);
  if (end != s.c_str() + s.size()) return false;
  *v = x;
  return true;
}

bool host_is_big_endian() {
  const union { uint32_t i; char c[4]; } probe = {0x01020304};
  return probe.c[0] == 1;
}

}  // namespace

extern "C" int chop_decode_pfm(const void* contents, size_t size, int64_t* height, int64_t* width, int64_t* channels,
                               float* image, size_t image_capacity, char* msg, size_t msg_capacity) {
  if (!contents || !height || !width || !channels) return CHOP_ERR_NULL;
  if (msg && msg_capacity) msg[0] = 0;
  const std::string input(static_cast<const char*>(contents), size);
  size_t pos = 0;
  size_t off = input.find_first_of(kWs, pos);
  if (off == std::string::npos) return fail(msg, msg_capacity, "no magic");
  const std::string magic = input.substr(pos, off - pos);
  if (magic != "Pf" && magic != "PF") return fail(msg, msg_capacity, "invalid format: " + magic);
  const int64_t ch = magic == "Pf" ? 1 : 3;

  off = input.find_first_not_of(kWs, off);
  if (off == std::string::npos) return fail(msg, msg_capacity, "no width");
  if (input[off] == '#')
    while (off < input.size() && input[off] != '\n') off++;
  pos = off;
  off = input.find_first_of(kWs, pos);
  if (off == std::string::npos) return fail(msg, msg_capacity, "no width");
  int64_t w = 0, h = 0;
  if (!parse_i64(input.substr(pos, off - pos), &w))
    return fail(msg, msg_capacity, "unable to parse width: " + input.substr(pos, off - pos));

  off = input.find_first_not_of(kWs, off);
  if (off == std::string::npos) return fail(msg, msg_capacity, "no height");
  pos = off;
  off = input.find_first_of(kWs, pos);
  if (off == std::string::npos) return fail(msg, msg_capacity, "no height");
  if (!parse_i64(input.substr(pos, off - pos), &h))
    return fail(msg, msg_capacity, "unable to parse height: " + input.substr(pos, off - pos));

  off = input.find_first_not_of(kWs, off);
  if (off == std::string::npos) return fail(msg, msg_capacity, "no scaling_factor");
  pos = off;
  off = input.find_first_of(kWs, pos);
  if (off == std::string::npos) return fail(msg, msg_capacity, "no scaling_factor");
  float scale = 0.f;
  if (!parse_f32(input.substr(pos, off - pos), &scale))
    return fail(msg, msg_capacity, "unable to parse scaling_factor: " + input.substr(pos, off - pos));
  if (host_is_big_endian() != (scale > 0.0f))   // the payload's byte order must be the host's
    return fail(msg, msg_capacity, "invalid scaling_factor value: mismatched endian type");
  if (w < 0 || h < 0) return fail(msg, msg_capacity, "negative image size");

  *height = h;
  *width = w;
  *channels = ch;
  off = off + 1;
  if (magic != "Pf") return fail(msg, msg_capacity, "no implement");
  // sizes from an untrusted header: compare by division, w * h * 4 may not fit 64 bits
  if (off > input.size() || (h != 0 && (uint64_t)w > (input.size() - off) / 4 / (uint64_t)h))
    return fail(msg, msg_capacity, "not enough data");
  const size_t n = (size_t)w * (size_t)h;
  if (!image) return CHOP_OK;
  if (image_capacity < n) return CHOP_ERR_WORKSPACE;
  const char* data = input.data() + off;
  for (int64_t r = 0; r < h; ++r)   // PFM stores the bottom row first
    std::memcpy(image + (size_t)r * w, data + (size_t)(h - 1 - r) * w * 4, (size_t)w * 4);
  return CHOP_OK;
}
