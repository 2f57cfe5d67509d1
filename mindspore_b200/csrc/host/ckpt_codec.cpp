// Streaming writer / scanner for the `.ckpt` wire format (concatenated protobuf `Checkpoint` messages, one
// `Value{tag, TensorProto{dims, tensor_type, tensor_content}}` each; layout of
// mindspore/ccsrc/utils/checkpoint.proto:17-44).  The writer appends one value at a time straight from the
// caller's buffer, so saving a multi-GB tensor never builds a second copy in host memory; CRC32 is folded in as
// blocks are written.  The scanner indexes a file (tag, dims, type, content offset/length) without reading the
// tensor payloads, which lets a loader pull only the parameters (or slices) a rank needs.
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#define MSB_API extern "C" __attribute__((visibility("default")))

namespace {

uint32_t g_crc_table[256];
bool g_crc_init = false;

void crc_init() {
  if (g_crc_init) return;
  for (uint32_t i = 0; i < 256; ++i) {
    uint32_t c = i;
    for (int k = 0; k < 8; ++k) c = (c & 1) ? 0xEDB88320u ^ (c >> 1) : c >> 1;
    g_crc_table[i] = c;
  }
  g_crc_init = true;
}

uint32_t crc_update(uint32_t crc, const uint8_t* p, size_t n) {
  crc_init();
  crc = ~crc;
  for (size_t i = 0; i < n; ++i) crc = g_crc_table[(crc ^ p[i]) & 0xFF] ^ (crc >> 8);
  return ~crc;
}

void put_varint(std::string* s, uint64_t v) {
  while (v >= 0x80) {
    s->push_back(static_cast<char>(v | 0x80));
    v >>= 7;
  }
  s->push_back(static_cast<char>(v));
}

size_t varint_len(uint64_t v) {
  size_t n = 1;
  while (v >= 0x80) { v >>= 7; ++n; }
  return n;
}

bool get_varint(const uint8_t* p, size_t n, size_t* pos, uint64_t* out) {
  uint64_t v = 0;
  int shift = 0;
  while (*pos < n) {
    const uint8_t b = p[(*pos)++];
    v |= static_cast<uint64_t>(b & 0x7F) << shift;
    if (!(b & 0x80)) { *out = v; return true; }
    shift += 7;
    if (shift > 63) return false;
  }
  return false;
}

}  // namespace

MSB_API uint32_t msb_crc32(uint32_t crc, const void* data, uint64_t len) {
  return crc_update(crc, static_cast<const uint8_t*>(data), static_cast<size_t>(len));
}

// Appends Checkpoint{value{tag, tensor{dims, type, content}}} to `path`.  crc_inout (may be null) is updated with
// the bytes written.  Returns bytes written, or -1.
MSB_API int64_t msb_ckpt_append_value(const char* path, const char* tag, const int64_t* dims, int n_dims,
                                      const char* type_name, const void* content, uint64_t content_len,
                                      uint32_t* crc_inout) {
  std::string tensor_hdr;
  for (int i = 0; i < n_dims; ++i) {
    tensor_hdr.push_back(0x08);
    put_varint(&tensor_hdr, static_cast<uint64_t>(dims[i]));
  }
  const size_t tlen = std::strlen(type_name);
  tensor_hdr.push_back(0x12);
  put_varint(&tensor_hdr, tlen);
  tensor_hdr.append(type_name, tlen);
  tensor_hdr.push_back(0x1a);
  put_varint(&tensor_hdr, content_len);
  const uint64_t tensor_len = tensor_hdr.size() + content_len;
  std::string value_hdr;
  const size_t taglen = std::strlen(tag);
  value_hdr.push_back(0x0a);
  put_varint(&value_hdr, taglen);
  value_hdr.append(tag, taglen);
  value_hdr.push_back(0x12);
  put_varint(&value_hdr, tensor_len);
  const uint64_t value_len = value_hdr.size() + tensor_len;
  std::string head;
  head.push_back(0x0a);
  put_varint(&head, value_len);
  head += value_hdr;
  head += tensor_hdr;
  FILE* f = std::fopen(path, "ab");
  if (!f) return -1;
  bool ok = std::fwrite(head.data(), 1, head.size(), f) == head.size();
  if (ok && content_len) ok = std::fwrite(content, 1, content_len, f) == content_len;
  std::fclose(f);
  if (!ok) return -1;
  if (crc_inout) {
    *crc_inout = crc_update(*crc_inout, reinterpret_cast<const uint8_t*>(head.data()), head.size());
    *crc_inout = crc_update(*crc_inout, static_cast<const uint8_t*>(content), content_len);
  }
  (void)varint_len;
  return static_cast<int64_t>(head.size() + content_len);
}

// Indexes an in-memory checkpoint image.  For record r: rec_out[4r..4r+3] = {tag offset, tag length,
// content offset, content length}; dims are appended to dims_out with dims_index_out[2r] = first index and
// dims_index_out[2r+1] = count; type names go to types_out as fixed 16-byte, NUL-padded fields.
// Returns the number of records, -1 if capacity is too small, -2 if the image is corrupt.
MSB_API int msb_ckpt_scan(const uint8_t* data, uint64_t len, int max_records, int64_t* rec_out, int64_t* dims_out,
                          int max_dims, int32_t* dims_index_out, char* types_out) {
  size_t pos = 0;
  int nrec = 0, ndim = 0;
  while (pos < len) {
    uint64_t key, vlen;
    if (!get_varint(data, len, &pos, &key) || key != 0x0a || !get_varint(data, len, &pos, &vlen)) return -2;
    const size_t vend = pos + vlen;
    if (vend > len) return -2;
    if (nrec >= max_records) return -1;
    int64_t* rec = rec_out + 4 * nrec;
    rec[0] = rec[1] = rec[2] = rec[3] = 0;
    dims_index_out[2 * nrec] = ndim;
    dims_index_out[2 * nrec + 1] = 0;
    std::memset(types_out + 16 * nrec, 0, 16);
    while (pos < vend) {
      uint64_t k, l;
      if (!get_varint(data, len, &pos, &k) || !get_varint(data, len, &pos, &l)) return -2;
      if (k == 0x0a) {
        rec[0] = static_cast<int64_t>(pos);
        rec[1] = static_cast<int64_t>(l);
        pos += l;
      } else if (k == 0x12) {
        const size_t tend = pos + l;
        while (pos < tend) {
          uint64_t kk;
          if (!get_varint(data, len, &pos, &kk)) return -2;
          if (kk == 0x08) {
            uint64_t d;
            if (!get_varint(data, len, &pos, &d)) return -2;
            if (ndim >= max_dims) return -1;
            dims_out[ndim++] = static_cast<int64_t>(d);
            dims_index_out[2 * nrec + 1] += 1;
          } else {
            uint64_t l3;
            if (!get_varint(data, len, &pos, &l3)) return -2;
            if (kk == 0x12) {
              std::memcpy(types_out + 16 * nrec, data + pos, l3 < 15 ? l3 : 15);
            } else if (kk == 0x1a) {
              rec[2] = static_cast<int64_t>(pos);
              rec[3] = static_cast<int64_t>(l3);
            } else if (kk == 0x0a) {  // packed dims
              size_t p2 = pos;
              while (p2 < pos + l3) {
                uint64_t d;
                if (!get_varint(data, len, &p2, &d)) return -2;
                if (ndim >= max_dims) return -1;
                dims_out[ndim++] = static_cast<int64_t>(d);
                dims_index_out[2 * nrec + 1] += 1;
              }
            }
            pos += l3;
          }
        }
      } else {
        pos += l;
      }
    }
    ++nrec;
    pos = vend;
  }
  return nrec;
}
