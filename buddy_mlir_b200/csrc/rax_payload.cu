// Reader for the payload section of a buddy-mlir .rax package (host code only).
//
// A .rax file is a FlatBuffer manifest (file identifier "RAX0") optionally
// followed by embedded payload blobs, an index and a 64-byte footer
// (runtime/include/buddy/runtime/core/ModelManifest.h:124-145 the structures,
// :202-246 the footer, :248-310 the index):
//   [manifest][payload blobs][index][footer]
//   footer : "RAXPAY01", u64 manifest_size @8, payload_offset @16 (= manifest_size),
//            payload_size @24, index_offset @32, index_size @40, flags @48   (little endian)
//   index  : "RAXIDX01", u32 version (1) @8, u32 count @12, then per entry
//            u16 kind @0, u32 name_size @4, u64 file_offset @8, u64 file_size @16, name bytes
// The manifest itself needs FlatBuffers to parse and is left alone; the payload
// entries are named (the weight blobs keep their file names, e.g.
// arg0-w8a32-f32.data), which is enough to pull the weights of a packaged model
// straight out of the package.  The checks are those of the reference reader.
#include "common.cuh"

#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

struct b200_rax {
  std::string path;
  uint64_t file_size = 0, manifest_size = 0, payload_offset = 0, payload_size = 0, flags = 0;
  struct Entry {
    int kind;
    std::string name;
    uint64_t offset, size;
  };
  std::vector<Entry> entries;
};

namespace {
using namespace b200;
uint64_t u64le(const uint8_t *p) {
  uint64_t v = 0;
  for (int i = 0; i < 8; ++i)
    v |= (uint64_t)p[i] << (8 * i);
  return v;
}
uint32_t u32le(const uint8_t *p) { return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24); }
bool read_range(FILE *f, uint64_t off, uint64_t n, std::vector<uint8_t> &out) {
  out.resize((size_t)n);
  if (fseeko(f, (off_t)off, SEEK_SET) != 0)
    return false;
  return n == 0 || fread(out.data(), 1, (size_t)n, f) == (size_t)n;
}
} // namespace

extern "C" {

int b200_rax_open(const char *path, b200_rax **out) {
  if (!path || !out)
    return fail(B200_EINVAL, "rax_open: null argument");
  FILE *f = fopen(path, "rb");
  if (!f)
    return fail(B200_EINVAL, "rax_open: cannot open %s", path);
  b200_rax *r = new b200_rax();
  r->path = path;
  auto bail = [&](const char *why) {
    fclose(f);
    delete r;
    return fail(B200_EINVAL, "rax_open(%s): %s", path, why);
  };
  fseeko(f, 0, SEEK_END);
  r->file_size = (uint64_t)ftello(f);
  std::vector<uint8_t> buf;
  if (r->file_size < 8 || !read_range(f, 0, 8, buf) || memcmp(buf.data() + 4, "RAX0", 4) != 0)
    return bail("not a RAX0 file");
  r->manifest_size = r->file_size;
  if (r->file_size >= 64 && read_range(f, r->file_size - 64, 64, buf) && memcmp(buf.data(), "RAXPAY01", 8) == 0) {
    const uint64_t fs = r->file_size;
    r->manifest_size = u64le(buf.data() + 8);
    r->payload_offset = u64le(buf.data() + 16);
    r->payload_size = u64le(buf.data() + 24);
    const uint64_t index_offset = u64le(buf.data() + 32), index_size = u64le(buf.data() + 40);
    r->flags = u64le(buf.data() + 48);
    if (r->manifest_size == 0 || r->manifest_size > fs)
      return bail("invalid payload footer (manifest_size)");
    if (r->payload_offset > fs || r->payload_size > fs - r->payload_offset)
      return bail("invalid payload footer (payload range)");
    if (index_offset > fs || index_size > fs - index_offset || index_offset + index_size > fs - 64)
      return bail("invalid payload footer (index range)");
    if (r->payload_offset != r->manifest_size)
      return bail("payload layout mismatch (payload_offset != manifest_size)");
    std::vector<uint8_t> idx;
    if (index_size < 16 || !read_range(f, index_offset, index_size, idx) || memcmp(idx.data(), "RAXIDX01", 8) != 0)
      return bail("payload index magic mismatch");
    if (u32le(idx.data() + 8) != 1)
      return bail("unsupported payload index version");
    const uint32_t count = u32le(idx.data() + 12);
    size_t cur = 16;
    for (uint32_t i = 0; i < count; ++i) {
      if (cur + 24 > idx.size())
        return bail("truncated payload index entry header");
      b200_rax::Entry e;
      e.kind = (int)((uint32_t)idx[cur] | ((uint32_t)idx[cur + 1] << 8));
      const uint32_t name_size = u32le(idx.data() + cur + 4);
      e.offset = u64le(idx.data() + cur + 8);
      e.size = u64le(idx.data() + cur + 16);
      cur += 24;
      if (name_size == 0 || cur + name_size > idx.size())
        return bail("truncated payload index entry name");
      e.name.assign((const char *)idx.data() + cur, name_size);
      cur += name_size;
      for (const auto &o : r->entries)
        if (o.name == e.name)
          return bail("duplicate payload entry name");
      if (e.offset > fs || e.size > fs - e.offset)
        return bail("payload entry out of file bounds");
      if (e.offset < r->payload_offset || e.offset + e.size > r->payload_offset + r->payload_size)
        return bail("payload entry out of payload section");
      r->entries.push_back(e);
    }
  }
  fclose(f);
  *out = r;
  return B200_OK;
}

void b200_rax_close(b200_rax *r) { delete r; }

int b200_rax_count(const b200_rax *r) { return r ? (int)r->entries.size() : 0; }

uint64_t b200_rax_manifest_bytes(const b200_rax *r) { return r ? r->manifest_size : 0; }

int b200_rax_entry(const b200_rax *r, int i, char *name, int name_cap, int *kind, uint64_t *offset, uint64_t *size) {
  if (!r || i < 0 || i >= (int)r->entries.size())
    return fail(B200_EINVAL, "rax_entry: no such entry");
  const auto &e = r->entries[(size_t)i];
  if (name && name_cap > 0) {
    strncpy(name, e.name.c_str(), (size_t)name_cap - 1);
    name[name_cap - 1] = 0;
  }
  if (kind) *kind = e.kind;
  if (offset) *offset = e.offset;
  if (size) *size = e.size;
  return B200_OK;
}

int b200_rax_find(const b200_rax *r, const char *name_suffix) {
  if (!r || !name_suffix)
    return -1;
  const size_t n = strlen(name_suffix);
  for (size_t i = 0; i < r->entries.size(); ++i) {
    const std::string &s = r->entries[i].name;
    if (s.size() >= n && s.compare(s.size() - n, n, name_suffix) == 0)
      return (int)i;
  }
  return -1;
}

int b200_rax_read(const b200_rax *r, int i, void *dst, uint64_t bytes) {
  if (!r || !dst || i < 0 || i >= (int)r->entries.size())
    return fail(B200_EINVAL, "rax_read: bad argument");
  const auto &e = r->entries[(size_t)i];
  if (bytes != e.size)
    return fail(B200_EINVAL, "rax_read: entry %s holds %llu bytes, %llu asked", e.name.c_str(),
                (unsigned long long)e.size, (unsigned long long)bytes);
  FILE *f = fopen(r->path.c_str(), "rb");
  if (!f)
    return fail(B200_EINVAL, "rax_read: cannot reopen %s", r->path.c_str());
  const bool ok = fseeko(f, (off_t)e.offset, SEEK_SET) == 0 && fread(dst, 1, (size_t)bytes, f) == (size_t)bytes;
  fclose(f);
  return ok ? B200_OK : fail(B200_EINVAL, "rax_read: short read of %s", e.name.c_str());
}

} // extern "C"
