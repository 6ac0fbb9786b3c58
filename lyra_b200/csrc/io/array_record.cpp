// ArrayRecord token shards: a Riegeli-structured record container with a chunk-offset footer,
// written and read natively (the reference depends on the array_record / Riegeli C++ libraries
// through `ArrayRecordWriter(path, "group_size:1")` and Grain's ArrayRecordDataSource,
// data/prepare_climbmix.py:49-51, lyra/data.py:40,57).
//
// Container, as publicly specified for Riegeli "records" files:
//   * the file is cut into 64 KiB blocks; every block starts with a 24-byte block header
//     {hash, distance back to the interrupted chunk's start, distance forward to its end};
//   * chunks have a 40-byte header {hash, data_size, data_hash, type(1B)+num_records(7B),
//     decoded_data_size}; the first chunk is the signature chunk (type 's', empty);
//   * a simple record chunk (type 'r') holds: compression byte, varint length of the sizes
//     buffer, the sizes buffer (one varint per record), then the record bytes;
//   * hashes are HighwayHash-64 with the key "Riegeli/records\n" repeated.
// ArrayRecord layout on top: `group_size` records per chunk, then a footer chunk (type 'f' here)
// listing every data chunk's file offset as little-endian u64, then a postscript chunk in the
// last 64 KiB block holding {footer_offset, magic, reserved}.
// This writer stores records uncompressed; the reader also accepts zstd chunks when libzstd.so.1
// can be dlopen'ed. Hash verification on read is optional (off by default).
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <dlfcn.h>
#include <fcntl.h>
#include <string>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include <vector>

namespace {

// ------------------------------------------------------------------ HighwayHash-64 (portable)
struct HHState {
  uint64_t v0[4], v1[4], mul0[4], mul1[4];
};

inline uint64_t rd64(const uint8_t* p) {
  uint64_t v;
  memcpy(&v, p, 8);
  return v;
}

void hh_reset(HHState* s, const uint64_t key[4]) {
  const uint64_t m0[4] = {0xdbe6d5d5fe4cce2full, 0xa4093822299f31d0ull, 0x13198a2e03707344ull, 0x243f6a8885a308d3ull};
  const uint64_t m1[4] = {0x3bd39e10cb0ef593ull, 0xc0acf169b5f18a8cull, 0xbe5466cf34e90c6cull, 0x452821e638d01377ull};
  for (int i = 0; i < 4; ++i) {
    s->mul0[i] = m0[i];
    s->mul1[i] = m1[i];
    s->v0[i] = m0[i] ^ key[i];
    s->v1[i] = m1[i] ^ ((key[i] >> 32) | (key[i] << 32));
  }
}

inline void zipper(uint64_t v1, uint64_t v0, uint64_t* add1, uint64_t* add0) {
  *add0 += (((v0 & 0x00000000ff000000ull) | (v1 & 0x000000ff00000000ull)) >> 24) |
           (((v0 & 0x0000ff0000000000ull) | (v1 & 0x00ff000000000000ull)) >> 16) | (v0 & 0x0000000000ff0000ull) |
           ((v0 & 0x000000000000ff00ull) << 32) | ((v1 & 0xff00000000000000ull) >> 8) | (v0 << 56);
  *add1 += (((v1 & 0x00000000ff000000ull) | (v0 & 0x000000ff00000000ull)) >> 24) | (v1 & 0x0000000000ff0000ull) |
           ((v1 & 0x0000ff0000000000ull) >> 16) | ((v1 & 0x000000000000ff00ull) << 24) |
           ((v0 & 0x00ff000000000000ull) >> 8) | ((v1 & 0x00000000000000ffull) << 48) | (v0 & 0xff00000000000000ull);
}

void hh_update(HHState* s, const uint64_t lanes[4]) {
  for (int i = 0; i < 4; ++i) {
    s->v1[i] += s->mul0[i] + lanes[i];
    s->mul0[i] ^= (s->v1[i] & 0xffffffffull) * (s->v0[i] >> 32);
    s->v0[i] += s->mul1[i];
    s->mul1[i] ^= (s->v0[i] & 0xffffffffull) * (s->v1[i] >> 32);
  }
  zipper(s->v1[1], s->v1[0], &s->v0[1], &s->v0[0]);
  zipper(s->v1[3], s->v1[2], &s->v0[3], &s->v0[2]);
  zipper(s->v0[1], s->v0[0], &s->v1[1], &s->v1[0]);
  zipper(s->v0[3], s->v0[2], &s->v1[3], &s->v1[2]);
}

void hh_packet(HHState* s, const uint8_t* p) {
  uint64_t lanes[4] = {rd64(p), rd64(p + 8), rd64(p + 16), rd64(p + 24)};
  hh_update(s, lanes);
}

void hh_remainder(HHState* s, const uint8_t* bytes, size_t size_mod32) {
  const size_t size_mod4 = size_mod32 & 3;
  const uint8_t* remainder = bytes + (size_mod32 & ~size_t(3));
  uint8_t packet[32] = {0};
  for (int i = 0; i < 4; ++i) s->v0[i] += (uint64_t(size_mod32) << 32) + size_mod32;
  for (int i = 0; i < 4; ++i) {  // rotate both 32-bit halves left by size_mod32
    uint32_t lo = uint32_t(s->v1[i]), hi = uint32_t(s->v1[i] >> 32);
    if (size_mod32) {
      lo = (lo << size_mod32) | (lo >> (32 - size_mod32));
      hi = (hi << size_mod32) | (hi >> (32 - size_mod32));
    }
    s->v1[i] = (uint64_t(hi) << 32) | lo;
  }
  for (size_t i = 0; i < size_t(remainder - bytes); ++i) packet[i] = bytes[i];
  if (size_mod32 & 16) {
    for (int i = 0; i < 4; ++i) packet[28 + i] = remainder[i + size_mod4 - 4];
  } else if (size_mod4) {
    packet[16 + 0] = remainder[0];
    packet[16 + 1] = remainder[size_mod4 >> 1];
    packet[16 + 2] = remainder[size_mod4 - 1];
  }
  hh_packet(s, packet);
}

uint64_t hh_finalize64(HHState* s) {
  for (int r = 0; r < 4; ++r) {
    uint64_t perm[4] = {(s->v0[2] >> 32) | (s->v0[2] << 32), (s->v0[3] >> 32) | (s->v0[3] << 32),
                        (s->v0[0] >> 32) | (s->v0[0] << 32), (s->v0[1] >> 32) | (s->v0[1] << 32)};
    hh_update(s, perm);
  }
  return s->v0[0] + s->v1[0] + s->mul0[0] + s->mul1[0];
}

uint64_t riegeli_hash(const uint8_t* data, size_t n) {
  static const uint64_t key[4] = {0x2f696c6567656952ull, 0x0a7364726f636572ull, 0x2f696c6567656952ull, 0x0a7364726f636572ull};
  HHState s;
  hh_reset(&s, key);
  size_t i = 0;
  for (; i + 32 <= n; i += 32) hh_packet(&s, data + i);
  if (n & 31) hh_remainder(&s, data + i, n & 31);
  return hh_finalize64(&s);
}

// ------------------------------------------------------------------ block / chunk geometry
constexpr uint64_t kBlock = 65536, kBlockHeader = 24, kUsable = kBlock - kBlockHeader, kChunkHeader = 40;
constexpr uint64_t kPostscriptMagic = 0x71930e704fdae05eull;

inline uint64_t add_with_overhead(uint64_t pos, uint64_t length) {
  const uint64_t overhead_blocks = (length + (pos + kUsable - 1) % kBlock) / kUsable;
  return pos + length + overhead_blocks * kBlockHeader;
}
inline uint64_t round_up_chunk_boundary(uint64_t pos) {
  const uint64_t in_block = pos % kBlock;
  return (in_block > 0 && in_block < kBlockHeader) ? pos + (kBlockHeader - in_block) : pos;
}

inline void put64(uint8_t* p, uint64_t v) { memcpy(p, &v, 8); }

void put_varint(std::vector<uint8_t>& out, uint64_t v) {
  while (v >= 0x80) {
    out.push_back(uint8_t(v) | 0x80);
    v >>= 7;
  }
  out.push_back(uint8_t(v));
}
bool get_varint(const uint8_t*& p, const uint8_t* end, uint64_t* v) {
  uint64_t r = 0;
  for (int shift = 0; shift < 64 && p < end; shift += 7) {
    const uint8_t b = *p++;
    r |= uint64_t(b & 0x7f) << shift;
    if (!(b & 0x80)) {
      *v = r;
      return true;
    }
  }
  return false;
}

// ------------------------------------------------------------------ writer
struct Writer {
  FILE* f = nullptr;
  uint64_t pos = 0;
  int group_size = 1;
  std::vector<std::vector<uint8_t>> pending;
  std::vector<uint64_t> chunk_offsets;
  bool failed = false;

  void raw(const uint8_t* p, size_t n) {
    if (n && fwrite(p, 1, n, f) != n) failed = true;
    pos += n;
  }
  // Writes one chunk (header + data + padding), inserting block headers at 64 KiB boundaries.
  void write_chunk(uint8_t type, uint64_t num_records, uint64_t decoded_size, const std::vector<uint8_t>& data) {
    const uint64_t begin = pos;
    uint8_t header[kChunkHeader];
    put64(header + 8, data.size());
    put64(header + 16, riegeli_hash(data.data(), data.size()));
    put64(header + 24, uint64_t(type) | (num_records << 8));
    put64(header + 32, decoded_size);
    put64(header, riegeli_hash(header + 8, kChunkHeader - 8));
    const uint64_t end = std::max(add_with_overhead(begin, kChunkHeader + data.size()), round_up_chunk_boundary(begin + num_records));
    std::vector<uint8_t> logical(header, header + kChunkHeader);
    logical.insert(logical.end(), data.begin(), data.end());
    size_t off = 0;
    while (pos < end) {
      if (pos % kBlock == 0) {
        uint8_t bh[kBlockHeader];
        put64(bh + 8, pos - begin);
        put64(bh + 16, end - pos);
        put64(bh, riegeli_hash(bh + 8, 16));
        raw(bh, kBlockHeader);
        continue;
      }
      const uint64_t room = std::min<uint64_t>(kBlock - pos % kBlock, end - pos);
      const size_t take = size_t(std::min<uint64_t>(room, logical.size() - off));
      if (take) {
        raw(logical.data() + off, take);
        off += take;
      } else {  // padding
        std::vector<uint8_t> zeros(size_t(room), 0);
        raw(zeros.data(), zeros.size());
      }
    }
  }
  void flush_group() {
    if (pending.empty()) return;
    std::vector<uint8_t> sizes, data;
    uint64_t decoded = 0;
    for (auto& r : pending) {
      put_varint(sizes, r.size());
      decoded += r.size();
    }
    data.push_back(0);  // compression: none
    put_varint(data, sizes.size());
    data.insert(data.end(), sizes.begin(), sizes.end());
    for (auto& r : pending) data.insert(data.end(), r.begin(), r.end());
    chunk_offsets.push_back(pos);
    write_chunk('r', pending.size(), decoded, data);
    pending.clear();
  }
};

// ------------------------------------------------------------------ reader
typedef size_t (*ZstdDecompressFn)(void*, size_t, const void*, size_t);
typedef unsigned (*ZstdIsErrorFn)(size_t);

struct Zstd {
  ZstdDecompressFn decompress = nullptr;
  ZstdIsErrorFn is_error = nullptr;
  Zstd() {
    void* h = dlopen("libzstd.so.1", RTLD_NOW | RTLD_LOCAL);
    if (!h) return;
    decompress = reinterpret_cast<ZstdDecompressFn>(dlsym(h, "ZSTD_decompress"));
    is_error = reinterpret_cast<ZstdIsErrorFn>(dlsym(h, "ZSTD_isError"));
  }
};
Zstd& zstd() {
  static Zstd z;
  return z;
}

struct RecordRef {
  uint64_t chunk;   // index into chunks
  uint32_t in_chunk;
};

struct Reader {
  int fd = -1;
  const uint8_t* map = nullptr;
  uint64_t size = 0;
  std::vector<uint64_t> chunks;       // file offsets of data chunks
  std::vector<uint64_t> chunk_first;  // first record index of each chunk
  uint64_t num_records = 0;
  // one decoded chunk cached (sequential access pattern)
  uint64_t cached = ~0ull;
  std::vector<uint8_t> values;
  std::vector<uint64_t> rec_off;

  // Copies `n` logical bytes starting at file position `pos`, skipping block headers.
  bool read_logical(uint64_t pos, uint8_t* out, uint64_t n, uint64_t* end_pos = nullptr) const {
    while (n) {
      if (pos % kBlock == 0) pos += kBlockHeader;
      if (pos >= size) return false;
      const uint64_t room = std::min<uint64_t>(std::min<uint64_t>(kBlock - pos % kBlock, n), size - pos);
      memcpy(out, map + pos, room);
      out += room;
      pos += room;
      n -= room;
    }
    if (end_pos) *end_pos = pos;
    return true;
  }
  bool chunk_header(uint64_t begin, uint64_t* data_size, uint8_t* type, uint64_t* nrec, uint64_t* decoded, uint64_t* data_pos) const {
    uint8_t h[kChunkHeader];
    if (!read_logical(begin, h, kChunkHeader, data_pos)) return false;
    *data_size = rd64(h + 8);
    const uint64_t tn = rd64(h + 24);
    *type = uint8_t(tn & 0xff);
    *nrec = tn >> 8;
    *decoded = rd64(h + 32);
    return true;
  }
  static bool decode_buffer(uint8_t compression, const uint8_t* p, size_t n, std::vector<uint8_t>* out) {
    if (compression == 0) {
      out->assign(p, p + n);
      return true;
    }
    const uint8_t* q = p;
    uint64_t raw_size;
    if (!get_varint(q, p + n, &raw_size)) return false;
    if (compression == 'z' && zstd().decompress) {
      out->resize(raw_size);
      const size_t got = zstd().decompress(out->data(), raw_size, q, size_t(p + n - q));
      return !zstd().is_error(got) && got == raw_size;
    }
    return false;  // brotli / snappy are not supported
  }
  bool load_chunk(uint64_t ci) {
    if (cached == ci) return true;
    uint64_t data_size, nrec, decoded, data_pos;
    uint8_t type;
    if (!chunk_header(chunks[ci], &data_size, &type, &nrec, &decoded, &data_pos) || type != 'r') return false;
    std::vector<uint8_t> data(data_size);
    if (!read_logical(data_pos, data.data(), data_size)) return false;
    const uint8_t* p = data.data();
    const uint8_t* end = p + data.size();
    if (p >= end) return false;
    const uint8_t compression = *p++;
    uint64_t sizes_len;
    if (!get_varint(p, end, &sizes_len) || uint64_t(end - p) < sizes_len) return false;
    std::vector<uint8_t> sizes;
    if (!decode_buffer(compression, p, sizes_len, &sizes)) return false;
    p += sizes_len;
    if (!decode_buffer(compression, p, size_t(end - p), &values)) return false;
    rec_off.assign(1, 0);
    const uint8_t* sp = sizes.data();
    const uint8_t* se = sp + sizes.size();
    for (uint64_t i = 0; i < nrec; ++i) {
      uint64_t s;
      if (!get_varint(sp, se, &s)) return false;
      rec_off.push_back(rec_off.back() + s);
    }
    if (rec_off.back() > values.size()) return false;
    cached = ci;
    return true;
  }
  bool locate(uint64_t idx, uint64_t* ci, uint64_t* local) const {
    if (idx >= num_records) return false;
    auto it = std::upper_bound(chunk_first.begin(), chunk_first.end(), idx);
    *ci = uint64_t(it - chunk_first.begin()) - 1;
    *local = idx - chunk_first[*ci];
    return true;
  }
  // Index from the postscript + footer; falls back to scanning the chunks from the start.
  bool build_index() {
    bool have = false;
    if (size >= kBlock) {
      const uint64_t ps = (size - 1) / kBlock * kBlock;  // postscript chunk starts at the last block boundary
      uint64_t data_size, nrec, decoded, data_pos;
      uint8_t type;
      if (chunk_header(ps, &data_size, &type, &nrec, &decoded, &data_pos) && data_size == 24) {
        uint8_t d[24];
        if (read_logical(data_pos, d, 24) && rd64(d + 8) == kPostscriptMagic) {
          const uint64_t footer = rd64(d);
          if (chunk_header(footer, &data_size, &type, &nrec, &decoded, &data_pos) && data_size % 8 == 0) {
            std::vector<uint8_t> f(data_size);
            if (read_logical(data_pos, f.data(), data_size)) {
              for (uint64_t i = 0; i < data_size / 8; ++i) chunks.push_back(rd64(f.data() + 8 * i));
              have = true;
            }
          }
        }
      }
    }
    if (!have) {  // sequential scan
      uint64_t pos = 0;
      while (pos < size) {
        uint64_t data_size, nrec, decoded, data_pos;
        uint8_t type;
        if (!chunk_header(pos, &data_size, &type, &nrec, &decoded, &data_pos)) break;
        if (type == 'r') chunks.push_back(pos);
        const uint64_t end = std::max(add_with_overhead(pos, kChunkHeader + data_size), round_up_chunk_boundary(pos + nrec));
        if (end <= pos) break;
        pos = end;
      }
    }
    chunk_first.clear();
    num_records = 0;
    for (uint64_t c : chunks) {
      uint64_t data_size, nrec, decoded, data_pos;
      uint8_t type;
      if (!chunk_header(c, &data_size, &type, &nrec, &decoded, &data_pos) || type != 'r') return false;
      chunk_first.push_back(num_records);
      num_records += nrec;
    }
    return true;
  }
};

}  // namespace

extern "C" {

void* lyra_ar_writer_open(const char* path, int group_size) {
  FILE* f = fopen(path, "wb");
  if (!f) return nullptr;
  Writer* w = new Writer;
  w->f = f;
  w->group_size = group_size > 0 ? group_size : 1;
  w->write_chunk('s', 0, 0, {});  // file signature
  return w;
}

int lyra_ar_writer_write(void* handle, const void* data, long long nbytes) {
  Writer* w = static_cast<Writer*>(handle);
  const uint8_t* p = static_cast<const uint8_t*>(data);
  w->pending.emplace_back(p, p + nbytes);
  if (int(w->pending.size()) >= w->group_size) w->flush_group();
  return w->failed ? -1 : 0;
}

int lyra_ar_writer_close(void* handle) {
  Writer* w = static_cast<Writer*>(handle);
  w->flush_group();
  // footer: offsets of all data chunks
  std::vector<uint8_t> footer(w->chunk_offsets.size() * 8);
  for (size_t i = 0; i < w->chunk_offsets.size(); ++i) put64(footer.data() + 8 * i, w->chunk_offsets[i]);
  const uint64_t footer_pos = w->pos;
  w->write_chunk('f', 0, footer.size(), footer);
  // pad to the next block boundary, then the postscript chunk opens the last block
  if (w->pos % kBlock) {
    std::vector<uint8_t> pad(size_t(kBlock - w->pos % kBlock), 0);
    w->raw(pad.data(), pad.size());
  }
  std::vector<uint8_t> ps(24, 0);
  put64(ps.data(), footer_pos);
  put64(ps.data() + 8, kPostscriptMagic);
  w->write_chunk('p', 0, ps.size(), ps);
  const bool ok = !w->failed && fclose(w->f) == 0;
  delete w;
  return ok ? 0 : -1;
}

void* lyra_ar_reader_open(const char* path) {
  int fd = ::open(path, O_RDONLY);
  if (fd < 0) return nullptr;
  struct stat st;
  if (fstat(fd, &st) != 0 || st.st_size == 0) {
    ::close(fd);
    return nullptr;
  }
  void* m = mmap(nullptr, size_t(st.st_size), PROT_READ, MAP_PRIVATE, fd, 0);
  if (m == MAP_FAILED) {
    ::close(fd);
    return nullptr;
  }
  Reader* r = new Reader;
  r->fd = fd;
  r->map = static_cast<const uint8_t*>(m);
  r->size = uint64_t(st.st_size);
  if (!r->build_index()) {
    munmap(m, size_t(st.st_size));
    ::close(fd);
    delete r;
    return nullptr;
  }
  return r;
}

long long lyra_ar_reader_num_records(void* handle) { return (long long)static_cast<Reader*>(handle)->num_records; }

long long lyra_ar_reader_record_size(void* handle, long long idx) {
  Reader* r = static_cast<Reader*>(handle);
  uint64_t ci, local;
  if (!r->locate(uint64_t(idx), &ci, &local) || !r->load_chunk(ci)) return -1;
  return (long long)(r->rec_off[local + 1] - r->rec_off[local]);
}

// Copies bytes [offset, offset + n) of record idx into out. Returns bytes copied or -1.
long long lyra_ar_reader_read(void* handle, long long idx, long long offset, long long n, void* out) {
  Reader* r = static_cast<Reader*>(handle);
  uint64_t ci, local;
  if (!r->locate(uint64_t(idx), &ci, &local) || !r->load_chunk(ci)) return -1;
  const uint64_t b = r->rec_off[local], e = r->rec_off[local + 1];
  if (uint64_t(offset) > e - b) return -1;
  const uint64_t take = std::min<uint64_t>(uint64_t(n), e - b - uint64_t(offset));
  memcpy(out, r->values.data() + b + offset, take);
  return (long long)take;
}

void lyra_ar_reader_close(void* handle) {
  Reader* r = static_cast<Reader*>(handle);
  munmap(const_cast<uint8_t*>(r->map), size_t(r->size));
  ::close(r->fd);
  delete r;
}

unsigned long long lyra_riegeli_hash(const void* data, long long n) { return riegeli_hash(static_cast<const uint8_t*>(data), size_t(n)); }

}  // extern "C"
