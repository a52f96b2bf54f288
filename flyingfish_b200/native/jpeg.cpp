// Baseline / extended-sequential JPEG decoder (8-bit, Huffman) for the image inputs of the server:
// grayscale, YCbCr (any sampling factors up to 4x4, e.g. 4:4:4, 4:2:2, 4:2:0), and four-component Adobe CMYK / YCCK
// files; restart intervals; 8- and 16-bit quantisation tables. Progressive, arithmetic-coded, lossless and 12-bit
// files are refused with an error code, as are images beyond the pixel limit given by the caller, before any
// allocation proportional to the image. Output: interleaved RGB bytes. The reference decodes JPEG data URLs through
// an image crate (src/serve/image.rs:2216-2250); this is an independent implementation of ITU-T T.81 decoding with a
// separable floating-point inverse DCT and replicated chroma upsampling.
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <vector>

namespace {

enum : int {
  JPEG_OK = 0, JPEG_TRUNCATED = -1, JPEG_NOT_JPEG = -2, JPEG_UNSUPPORTED = -3, JPEG_BAD_TABLE = -4, JPEG_BAD_STREAM = -5,
  JPEG_TOO_LARGE = -6, JPEG_SMALL_BUFFER = -7,
};

const uint8_t ZIGZAG[64] = {0,  1,  8,  16, 9,  2,  3,  10, 17, 24, 32, 25, 18, 11, 4,  5,  12, 19, 26, 33, 40, 48,
                            41, 34, 27, 20, 13, 6,  7,  14, 21, 28, 35, 42, 49, 56, 57, 50, 43, 36, 29, 22, 15, 23,
                            30, 37, 44, 51, 58, 59, 52, 45, 38, 31, 39, 46, 53, 60, 61, 54, 47, 55, 62, 63};

struct Huff {
  bool present = false;
  uint8_t vals[256];
  int mincode[17], maxcode[18], valptr[17];
  // 9-bit look-ahead: (length << 8) | value, 0 = longer code
  uint16_t fast[512];
};

struct Component {
  int id = 0, h = 1, v = 1, tq = 0, td = 0, ta = 0;
  int blocks_w = 0, blocks_h = 0;      // padded to whole MCUs
  std::vector<uint8_t> plane;          // blocks_w * 8 x blocks_h * 8
  int pred = 0;
};

struct Reader {
  const uint8_t* p; size_t n, pos = 0;
  uint32_t bits = 0; int nbits = 0; bool hit_marker = false;
  bool fill() {
    while (nbits <= 24) {
      if (hit_marker || pos >= n) { bits |= 0; nbits += 8; hit_marker = true; continue; }   // feed zeros past the data
      uint8_t b = p[pos];
      if (b == 0xFF) {
        if (pos + 1 >= n) { hit_marker = true; continue; }
        const uint8_t m = p[pos + 1];
        if (m == 0x00) { pos += 2; }
        else { hit_marker = true; continue; }          // a marker: leave it for the caller
      } else {
        pos += 1;
      }
      bits |= (uint32_t)b << (24 - nbits);
      nbits += 8;
    }
    return true;
  }
  int peek(int k) { fill(); return (int)(bits >> (32 - k)); }
  void skip(int k) { bits <<= k; nbits -= k; }
  int get(int k) { if (k == 0) return 0; const int v = peek(k); skip(k); return v; }
  void reset_bits() { bits = 0; nbits = 0; hit_marker = false; }
};

bool build_huff(Huff& h, const uint8_t counts[16], const uint8_t* vals, int nvals) {
  int code = 0, k = 0;
  std::memset(h.fast, 0, sizeof(h.fast));
  for (int len = 1; len <= 16; ++len) {
    h.valptr[len] = k;
    h.mincode[len] = code;
    for (int i = 0; i < counts[len - 1]; ++i, ++k, ++code) {
      if (k >= nvals) return false;
      if (len <= 9) {
        const int first = code << (9 - len);
        for (int f = 0; f < (1 << (9 - len)); ++f) h.fast[first + f] = (uint16_t)((len << 8) | vals[k]);
      }
    }
    h.maxcode[len] = counts[len - 1] ? code - 1 : -1;
    if (code > (1 << len)) return false;
    code <<= 1;
  }
  h.maxcode[17] = 0x7fffffff;
  std::memcpy(h.vals, vals, nvals);
  h.present = true;
  return true;
}

inline int decode_symbol(Reader& r, const Huff& h) {
  const int look = r.peek(9);
  const uint16_t f = h.fast[look];
  if (f) { r.skip(f >> 8); return f & 0xff; }
  int code = r.peek(16);
  for (int len = 10; len <= 16; ++len) {
    const int c = code >> (16 - len);
    if (h.maxcode[len] >= 0 && c <= h.maxcode[len] && c >= h.mincode[len]) {
      r.skip(len);
      return h.vals[h.valptr[len] + c - h.mincode[len]];
    }
  }
  return -1;
}

inline int extend(int v, int t) { return v < (1 << (t - 1)) ? v - (1 << t) + 1 : v; }

void idct8x8(const float* in, uint8_t* out, int stride) {
  static float C[8][8];
  static bool init = false;
  if (!init) {
    for (int x = 0; x < 8; ++x)
      for (int u = 0; u < 8; ++u)
        C[x][u] = (u == 0 ? std::sqrt(0.125f) : 0.5f) * std::cos((2 * x + 1) * u * 3.14159265358979323846f / 16.0f);
    init = true;
  }
  float tmp[64];
  for (int y = 0; y < 8; ++y)            // rows: tmp[y][x] = sum_u C[x][u] in[y][u]
    for (int x = 0; x < 8; ++x) {
      float s = 0.f;
      for (int u = 0; u < 8; ++u) s += C[x][u] * in[y * 8 + u];
      tmp[y * 8 + x] = s;
    }
  for (int x = 0; x < 8; ++x)
    for (int y = 0; y < 8; ++y) {
      float s = 0.f;
      for (int v = 0; v < 8; ++v) s += C[y][v] * tmp[v * 8 + x];
      const int q = (int)std::lrintf(s + 128.f);
      out[y * stride + x] = (uint8_t)(q < 0 ? 0 : q > 255 ? 255 : q);
    }
}

struct Decoder {
  const uint8_t* data; size_t n;
  int width = 0, height = 0, ncomp = 0;
  uint16_t qt[4][64]; bool qt_present[4] = {false, false, false, false};
  Huff dc[4], ac[4];
  Component comp[4];
  int restart = 0, hmax = 1, vmax = 1;
  bool adobe = false; int adobe_transform = -1;
  bool have_frame = false;

  static int be16(const uint8_t* p) { return (p[0] << 8) | p[1]; }

  int parse_headers(size_t& pos, bool stop_at_frame, long long max_pixels) {
    if (n < 4 || data[0] != 0xFF || data[1] != 0xD8) return JPEG_NOT_JPEG;
    pos = 2;
    while (true) {
      if (pos + 4 > n) return JPEG_TRUNCATED;
      if (data[pos] != 0xFF) return JPEG_BAD_STREAM;
      while (pos < n && data[pos] == 0xFF) ++pos;                 // fill bytes
      if (pos >= n) return JPEG_TRUNCATED;
      const int m = data[pos++];
      if (m == 0xD8 || (m >= 0xD0 && m <= 0xD7) || m == 0x01) continue;
      if (m == 0xD9) return JPEG_BAD_STREAM;
      if (pos + 2 > n) return JPEG_TRUNCATED;
      const int len = be16(data + pos);
      if (len < 2 || pos + len > n) return JPEG_TRUNCATED;
      const uint8_t* seg = data + pos + 2;
      const int sl = len - 2;
      if (m == 0xDB) {
        int o = 0;
        while (o < sl) {
          const int pq = seg[o] >> 4, tq = seg[o] & 15;
          if (tq > 3 || pq > 1) return JPEG_BAD_TABLE;
          ++o;
          if (o + 64 * (pq + 1) > sl) return JPEG_TRUNCATED;
          for (int i = 0; i < 64; ++i) { qt[tq][ZIGZAG[i]] = pq ? (uint16_t)be16(seg + o + 2 * i) : seg[o + i]; }
          o += 64 * (pq + 1);
          qt_present[tq] = true;
        }
      } else if (m == 0xC4) {
        int o = 0;
        while (o < sl) {
          if (o + 17 > sl) return JPEG_TRUNCATED;
          const int tc = seg[o] >> 4, th = seg[o] & 15;
          if (tc > 1 || th > 3) return JPEG_BAD_TABLE;
          int total = 0;
          for (int i = 0; i < 16; ++i) total += seg[o + 1 + i];
          if (total > 256 || o + 17 + total > sl) return JPEG_BAD_TABLE;
          if (!build_huff(tc ? ac[th] : dc[th], seg + o + 1, seg + o + 17, total)) return JPEG_BAD_TABLE;
          o += 17 + total;
        }
      } else if (m == 0xC0 || m == 0xC1) {
        if (sl < 6 || seg[0] != 8) return JPEG_UNSUPPORTED;
        height = be16(seg + 1); width = be16(seg + 3); ncomp = seg[5];
        if (width <= 0 || height <= 0 || (ncomp != 1 && ncomp != 3 && ncomp != 4) || sl < 6 + 3 * ncomp) return JPEG_UNSUPPORTED;
        if ((long long)width * height > max_pixels) return JPEG_TOO_LARGE;
        for (int i = 0; i < ncomp; ++i) {
          comp[i].id = seg[6 + 3 * i]; comp[i].h = seg[7 + 3 * i] >> 4; comp[i].v = seg[7 + 3 * i] & 15; comp[i].tq = seg[8 + 3 * i];
          if (comp[i].h < 1 || comp[i].h > 4 || comp[i].v < 1 || comp[i].v > 4 || comp[i].tq > 3) return JPEG_UNSUPPORTED;
          if (comp[i].h > hmax) hmax = comp[i].h;
          if (comp[i].v > vmax) vmax = comp[i].v;
        }
        have_frame = true;
        if (stop_at_frame) return JPEG_OK;
      } else if (m == 0xC2 || m == 0xC3 || (m >= 0xC5 && m <= 0xCF && m != 0xC8)) {
        return JPEG_UNSUPPORTED;                                   // progressive, lossless, arithmetic, differential
      } else if (m == 0xDD) {
        if (sl < 2) return JPEG_TRUNCATED;
        restart = be16(seg);
      } else if (m == 0xEE) {
        if (sl >= 12 && std::memcmp(seg, "Adobe", 5) == 0) { adobe = true; adobe_transform = seg[11]; }
      } else if (m == 0xDA) {
        if (!have_frame) return JPEG_BAD_STREAM;
        if (sl < 1 || seg[0] != ncomp || sl < 1 + 2 * ncomp + 3) return JPEG_UNSUPPORTED;   // one interleaved scan
        for (int i = 0; i < ncomp; ++i) {
          const int cid = seg[1 + 2 * i];
          int j = 0;
          while (j < ncomp && comp[j].id != cid) ++j;
          if (j == ncomp) return JPEG_BAD_STREAM;
          comp[j].td = seg[2 + 2 * i] >> 4; comp[j].ta = seg[2 + 2 * i] & 15;
          if (comp[j].td > 3 || comp[j].ta > 3) return JPEG_BAD_TABLE;
        }
        pos += len;
        return JPEG_OK;
      }
      pos += len;
    }
  }

  int decode_scan(size_t pos) {
    const int mcu_w = 8 * hmax, mcu_h = 8 * vmax;
    const int mcus_x = (width + mcu_w - 1) / mcu_w, mcus_y = (height + mcu_h - 1) / mcu_h;
    for (int i = 0; i < ncomp; ++i) {
      Component& c = comp[i];
      if (!qt_present[c.tq] || !dc[c.td].present || !ac[c.ta].present) return JPEG_BAD_TABLE;
      c.blocks_w = mcus_x * c.h; c.blocks_h = mcus_y * c.v;
      c.plane.assign((size_t)c.blocks_w * 8 * c.blocks_h * 8, 0);
      c.pred = 0;
    }
    Reader r{data, n, pos};
    int until_restart = restart, next_rst = 0;
    float block[64];
    for (int my = 0; my < mcus_y; ++my) {
      for (int mx = 0; mx < mcus_x; ++mx) {
        if (restart && until_restart == 0) {
          // byte-align, expect RSTn
          r.reset_bits();
          size_t q = r.pos;
          while (q + 1 < n && !(data[q] == 0xFF && data[q + 1] >= 0xD0 && data[q + 1] <= 0xD7)) ++q;
          if (q + 1 >= n) return JPEG_TRUNCATED;
          if (data[q + 1] != 0xD0 + next_rst) return JPEG_BAD_STREAM;
          next_rst = (next_rst + 1) & 7;
          r.pos = q + 2;
          for (int i = 0; i < ncomp; ++i) comp[i].pred = 0;
          until_restart = restart;
        }
        for (int i = 0; i < ncomp; ++i) {
          Component& c = comp[i];
          const int stride = c.blocks_w * 8;
          for (int by = 0; by < c.v; ++by) {
            for (int bx = 0; bx < c.h; ++bx) {
              std::memset(block, 0, sizeof(block));
              int t = decode_symbol(r, dc[c.td]);
              if (t < 0 || t > 11) return JPEG_BAD_STREAM;
              const int diff = t ? extend(r.get(t), t) : 0;
              c.pred += diff;
              block[0] = (float)(c.pred * (int)qt[c.tq][0]);
              for (int k = 1; k < 64;) {
                const int rs = decode_symbol(r, ac[c.ta]);
                if (rs < 0) return JPEG_BAD_STREAM;
                const int run = rs >> 4, sz = rs & 15;
                if (sz == 0) {
                  if (run == 15) { k += 16; continue; }
                  break;                                           // end of block
                }
                k += run;
                if (k > 63) return JPEG_BAD_STREAM;
                const int v = extend(r.get(sz), sz);
                block[ZIGZAG[k]] = (float)(v * (int)qt[c.tq][ZIGZAG[k]]);
                ++k;
              }
              uint8_t* dst = c.plane.data() + (size_t)((my * c.v + by) * 8) * stride + (mx * c.h + bx) * 8;
              idct8x8(block, dst, stride);
            }
          }
        }
        if (restart) --until_restart;
      }
    }
    return JPEG_OK;
  }

  inline uint8_t sample(const Component& c, int x, int y) const {
    const int sx = x * c.h / hmax, sy = y * c.v / vmax;
    return c.plane[(size_t)sy * c.blocks_w * 8 + sx];
  }

  void to_rgb(uint8_t* out) const {
    auto clamp = [](float v) { const int q = (int)std::lrintf(v); return (uint8_t)(q < 0 ? 0 : q > 255 ? 255 : q); };
    for (int y = 0; y < height; ++y) {
      for (int x = 0; x < width; ++x) {
        uint8_t* o = out + ((size_t)y * width + x) * 3;
        if (ncomp == 1) {
          o[0] = o[1] = o[2] = sample(comp[0], x, y);
        } else {
          const float a = sample(comp[0], x, y), b = sample(comp[1], x, y), c = sample(comp[2], x, y);
          const bool ycc = ncomp == 3 ? !(adobe && adobe_transform == 0) : (adobe_transform == 2);
          float r, g, bl;
          if (ycc) {
            r = a + 1.402f * (c - 128.f);
            g = a - 0.344136f * (b - 128.f) - 0.714136f * (c - 128.f);
            bl = a + 1.772f * (b - 128.f);
          } else {
            r = a; g = b; bl = c;
          }
          if (ncomp == 4) {
            // Adobe files store inverted CMYK: channel = 255 - ink; YCCK carries inverted CMY in the converted RGB
            const float k = sample(comp[3], x, y);
            r = r * k / 255.f; g = g * k / 255.f; bl = bl * k / 255.f;
          }
          o[0] = clamp(r); o[1] = clamp(g); o[2] = clamp(bl);
        }
      }
    }
  }
};

}  // namespace

#define FF_HOST_API __attribute__((visibility("default")))

extern "C" {

// Dimensions without decoding. Returns 0 or a negative error code.
FF_HOST_API int ff_jpeg_info(const uint8_t* data, size_t n, int* width, int* height, int* components) {
  Decoder d{data, n};
  size_t pos = 0;
  const int rc = d.parse_headers(pos, true, (long long)1 << 40);
  if (rc) return rc;
  if (width) *width = d.width;
  if (height) *height = d.height;
  if (components) *components = d.ncomp;
  return JPEG_OK;
}

// Decode to interleaved RGB. `out_bytes` must be at least width * height * 3; images with more than `max_pixels`
// pixels are refused before anything is allocated.
FF_HOST_API int ff_jpeg_decode(const uint8_t* data, size_t n, uint8_t* out, size_t out_bytes, long long max_pixels) {
  Decoder d{data, n};
  size_t pos = 0;
  int rc = d.parse_headers(pos, false, max_pixels);
  if (rc) return rc;
  if ((size_t)d.width * d.height * 3 > out_bytes) return JPEG_SMALL_BUFFER;
  rc = d.decode_scan(pos);
  if (rc) return rc;
  d.to_rgb(out);
  return JPEG_OK;
}

}  // extern "C"
