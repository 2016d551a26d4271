// Log-structured merge store: the durable key/value engine under the vector-index namespaces.
//
// Shape of the reference's engine (zig/pkg/antfly/src/storage/lsm/LSM.md "Preferred Design"; lsm_backend/wal.zig,
// compaction.zig, recovery.zig, storage_io.zig; the namespace interface of zig/lib/vectorindex/src/store.zig:104-278):
// a commit appends one framed record to a write-ahead log and applies it to a mutable in-memory table; a full table
// is rotated into an immutable queue; a background thread turns immutable tables into sorted table files and merges
// files level by level; a manifest names the live files and is replaced atomically.  Slow work (encoding, file
// writes, merges) runs outside the store mutex: select under the mutex, build outside, publish under it again.
// Readers pin a version (memory tables + file set) and a sequence number, so a read transaction sees one state for
// as long as it lives while writers and compactions carry on.
//
// File formats are this project's own:
//   wal-<n>.log    records  [u32 payload bytes][u32 crc32(payload)][payload]; payload = [u64 first sequence]
//                  then operations [u8 kind 1=put 2=delete][varint key bytes][varint value bytes][key][value]
//   <n>.tbl        data blocks of entries [u8 kind][varint key][varint value][key][value], each block followed by
//                  its crc32; an index block (last key, offset, bytes of every data block); a bloom filter over
//                  the keys (10 bits per key, 7 probes); a 64-byte footer with the offsets, counts and a magic
//   MANIFEST       text: one "file <level> <number> <bytes> <entries> <hex smallest> <hex largest>" line per live
//                  table, "next <file number>", "seq <last sequence>", "wal <oldest log still needed>"
// Keys carry their namespace as a first byte, so the four index namespaces share one ordered key space.
#include <algorithm>
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <shared_mutex>
#include <string>
#include <thread>
#include <vector>

#include <dirent.h>
#include <fcntl.h>
#include <sys/file.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

namespace {

using Bytes = std::string;

constexpr uint64_t kTableMagic = 0x4146424c534d5431ull;   // "AFBLSMT1"
constexpr int kLevels = 6;
constexpr uint8_t kPut = 1, kDel = 2;

// ---- small helpers ------------------------------------------------------------------------------------------
uint32_t crc32(const uint8_t* p, size_t n) {                        // slicing-by-8
  static uint32_t table[8][256];
  static std::once_flag once;
  std::call_once(once, [] {
    for (uint32_t i = 0; i < 256; ++i) {
      uint32_t c = i;
      for (int k = 0; k < 8; ++k) c = (c & 1) ? 0xEDB88320u ^ (c >> 1) : c >> 1;
      table[0][i] = c;
    }
    for (uint32_t i = 0; i < 256; ++i)
      for (int t = 1; t < 8; ++t) table[t][i] = table[0][table[t - 1][i] & 0xFF] ^ (table[t - 1][i] >> 8);
  });
  uint32_t c = 0xFFFFFFFFu;
  while (n >= 8) {
    uint32_t a, b;
    std::memcpy(&a, p, 4);
    std::memcpy(&b, p + 4, 4);
    a ^= c;
    c = table[7][a & 0xFF] ^ table[6][(a >> 8) & 0xFF] ^ table[5][(a >> 16) & 0xFF] ^ table[4][a >> 24] ^
        table[3][b & 0xFF] ^ table[2][(b >> 8) & 0xFF] ^ table[1][(b >> 16) & 0xFF] ^ table[0][b >> 24];
    p += 8; n -= 8;
  }
  for (size_t i = 0; i < n; ++i) c = table[0][(c ^ p[i]) & 0xFF] ^ (c >> 8);
  return c ^ 0xFFFFFFFFu;
}

void put_varint(Bytes& out, uint64_t v) {
  while (v >= 0x80) { out.push_back(char(v | 0x80)); v >>= 7; }
  out.push_back(char(v));
}

// Reads a varint from [p, end); returns nullptr when it runs off the end or is longer than ten bytes.
const uint8_t* get_varint(const uint8_t* p, const uint8_t* end, uint64_t* v) {
  uint64_t r = 0;
  for (int shift = 0; shift < 70 && p < end; shift += 7) {
    uint64_t b = *p++;
    r |= (b & 0x7F) << shift;
    if (!(b & 0x80)) { *v = r; return p; }
  }
  return nullptr;
}

template <class T> void put_fixed(Bytes& out, T v) { out.append(reinterpret_cast<const char*>(&v), sizeof v); }
template <class T> T get_fixed(const uint8_t* p) { T v; std::memcpy(&v, p, sizeof v); return v; }

uint64_t hash64(const char* p, size_t n, uint64_t seed) {          // FNV-1a, then a finaliser
  uint64_t h = 1469598103934665603ull ^ seed;
  for (size_t i = 0; i < n; ++i) { h ^= uint8_t(p[i]); h *= 1099511628211ull; }
  h ^= h >> 33; h *= 0xff51afd7ed558ccdull; h ^= h >> 33;
  return h;
}

bool write_all(int fd, const char* p, size_t n) {
  while (n) {
    ssize_t w = ::write(fd, p, n);
    if (w < 0) { if (errno == EINTR) continue; return false; }
    p += w; n -= size_t(w);
  }
  return true;
}

void sync_dir(const std::string& dir) {
  int fd = ::open(dir.c_str(), O_RDONLY | O_DIRECTORY);
  if (fd >= 0) { ::fsync(fd); ::close(fd); }
}

std::string hex(const Bytes& b) {
  static const char* d = "0123456789abcdef";
  std::string s;
  for (unsigned char c : b) { s.push_back(d[c >> 4]); s.push_back(d[c & 15]); }
  return s.empty() ? "-" : s;
}

Bytes unhex(const std::string& s) {
  Bytes b;
  if (s == "-") return b;
  auto v = [](char c) { return c <= '9' ? c - '0' : c - 'a' + 10; };
  for (size_t i = 0; i + 1 < s.size(); i += 2) b.push_back(char(v(s[i]) << 4 | v(s[i + 1])));
  return b;
}

int compare(const uint8_t* a, size_t an, const Bytes& b) {
  int c = std::memcmp(a, b.data(), std::min(an, b.size()));
  return c ? c : (an < b.size() ? -1 : an > b.size() ? 1 : 0);
}

// ---- table files --------------------------------------------------------------------------------------------
struct BlockHandle { Bytes last_key; uint64_t offset; uint32_t bytes; };

struct TableBuilder {
  std::string path;
  int fd = -1;
  Bytes block, index;
  std::vector<uint64_t> hashes;
  uint64_t offset = 0, entries = 0, blocks = 0;
  Bytes smallest, largest, last;
  size_t block_target;
  bool ok = true;

  TableBuilder(const std::string& p, size_t block_bytes) : path(p), block_target(block_bytes) {
    fd = ::open(p.c_str(), O_CREAT | O_TRUNC | O_WRONLY, 0644);
    ok = fd >= 0;
  }
  void add(const Bytes& key, uint8_t kind, const Bytes& value) {        // keys strictly ascending
    if (entries == 0) smallest = key;
    largest = last = key;
    block.push_back(char(kind));
    put_varint(block, key.size());
    put_varint(block, value.size());
    block += key;
    block += value;
    hashes.push_back(hash64(key.data(), key.size(), 0));
    ++entries;
    if (block.size() >= block_target) finish_block();
  }
  void finish_block() {
    if (block.empty()) return;
    put_varint(index, last.size());
    index += last;
    put_fixed<uint64_t>(index, offset);
    put_fixed<uint32_t>(index, uint32_t(block.size()));
    put_fixed<uint32_t>(block, crc32(reinterpret_cast<const uint8_t*>(block.data()), block.size()));
    ok = ok && write_all(fd, block.data(), block.size());
    offset += block.size();
    block.clear();
    ++blocks;
  }
  // Returns the file's size, or 0 on an IO error (the partial file is removed).
  uint64_t finish(bool sync) {
    finish_block();
    uint64_t index_off = offset;
    put_fixed<uint32_t>(index, crc32(reinterpret_cast<const uint8_t*>(index.data()), index.size()));
    ok = ok && write_all(fd, index.data(), index.size());
    offset += index.size();
    uint64_t bloom_off = offset;
    uint64_t bits = std::max<uint64_t>(64, entries * 10);
    bits = (bits + 63) / 64 * 64;
    Bytes bloom(bits / 8, '\0');
    for (uint64_t h : hashes) {
      uint64_t delta = (h >> 17) | (h << 47);
      for (int k = 0; k < 7; ++k) { uint64_t b = h % bits; bloom[b >> 3] |= char(1 << (b & 7)); h += delta; }
    }
    ok = ok && write_all(fd, bloom.data(), bloom.size());
    offset += bloom.size();
    Bytes foot;
    put_fixed<uint64_t>(foot, index_off);
    put_fixed<uint64_t>(foot, index.size());
    put_fixed<uint64_t>(foot, bloom_off);
    put_fixed<uint64_t>(foot, bloom.size());
    put_fixed<uint64_t>(foot, entries);
    put_fixed<uint64_t>(foot, blocks);
    put_fixed<uint64_t>(foot, uint64_t(crc32(reinterpret_cast<const uint8_t*>(bloom.data()), bloom.size())));
    put_fixed<uint64_t>(foot, kTableMagic);
    ok = ok && write_all(fd, foot.data(), foot.size());
    offset += foot.size();
    if (ok && sync) ok = ::fdatasync(fd) == 0;
    ::close(fd);
    fd = -1;
    if (!ok) { ::unlink(path.c_str()); return 0; }
    return offset;
  }
  ~TableBuilder() { if (fd >= 0) { ::close(fd); ::unlink(path.c_str()); } }
};

struct Entry { const uint8_t* key; uint32_t klen; const uint8_t* val; uint32_t vlen; uint8_t kind; };

// One open table file, mapped read-only.  Immutable after open(); shared by every version that lists it.  The file
// is unlinked when the last holder lets go of a table that a compaction made obsolete.
struct Table {
  std::string path;
  uint64_t number = 0, bytes = 0, entries = 0;
  int level = 0;
  Bytes smallest, largest;
  const uint8_t* map = nullptr;
  std::vector<BlockHandle> index;
  const uint8_t* bloom = nullptr;
  uint64_t bloom_bits = 0;
  std::atomic<bool> obsolete{false};
  mutable std::unique_ptr<std::atomic<uint8_t>[]> verified;            // per data block: checksum already checked
  mutable std::atomic<uint64_t> bloom_skips{0};

  ~Table() {
    if (map) ::munmap(const_cast<uint8_t*>(map), bytes);
    if (obsolete.load()) ::unlink(path.c_str());
  }

  // Empty string on success, else what is wrong with the file.
  std::string open(const std::string& p) {
    path = p;
    int fd = ::open(p.c_str(), O_RDONLY);
    if (fd < 0) return "cannot open " + p;
    struct stat st;
    if (::fstat(fd, &st) != 0 || st.st_size < 64) { ::close(fd); return p + ": shorter than a footer"; }
    bytes = uint64_t(st.st_size);
    void* m = ::mmap(nullptr, bytes, PROT_READ, MAP_SHARED, fd, 0);
    ::close(fd);
    if (m == MAP_FAILED) return "cannot map " + p;
    map = static_cast<const uint8_t*>(m);
    const uint8_t* f = map + bytes - 64;
    if (get_fixed<uint64_t>(f + 56) != kTableMagic) return p + ": not a table file (bad magic)";
    uint64_t ioff = get_fixed<uint64_t>(f), ilen = get_fixed<uint64_t>(f + 8), boff = get_fixed<uint64_t>(f + 16),
             blen = get_fixed<uint64_t>(f + 24), nblocks = get_fixed<uint64_t>(f + 40);
    entries = get_fixed<uint64_t>(f + 32);
    if (ilen < 4 || ioff > bytes || ilen > bytes - ioff || boff > bytes || blen > bytes - boff || blen % 8)
      return p + ": footer offsets outside the file";
    if (crc32(map + ioff, ilen - 4) != get_fixed<uint32_t>(map + ioff + ilen - 4)) return p + ": index checksum";
    if (uint64_t(crc32(map + boff, blen)) != get_fixed<uint64_t>(f + 48)) return p + ": filter checksum";
    const uint8_t *q = map + ioff, *end = map + ioff + ilen - 4;
    while (q < end) {
      uint64_t kl;
      q = get_varint(q, end, &kl);
      if (!q || kl > uint64_t(end - q) || uint64_t(end - q) - kl < 12) return p + ": index entry runs off its block";
      BlockHandle h;
      h.last_key.assign(reinterpret_cast<const char*>(q), kl);
      q += kl;
      h.offset = get_fixed<uint64_t>(q);
      h.bytes = get_fixed<uint32_t>(q + 8);
      q += 12;
      if (h.offset > ioff || uint64_t(h.bytes) + 4 > ioff - h.offset) return p + ": data block outside the file";
      index.push_back(std::move(h));
    }
    if (index.size() != nblocks) return p + ": block count does not match the index";
    verified.reset(new std::atomic<uint8_t>[index.size() + 1]);
    for (size_t i = 0; i <= index.size(); ++i) verified[i].store(0);
    bloom = map + boff;
    bloom_bits = blen * 8;
    if (!index.empty()) {
      largest = index.back().last_key;
      std::vector<uint32_t> offs;
      std::string err = parse_block(0, &offs);
      if (!err.empty()) return err;
      if (!offs.empty()) { Entry e = entry_at(0, offs[0]); smallest.assign(reinterpret_cast<const char*>(e.key), e.klen); }
    }
    return "";
  }

  bool may_contain(const Bytes& key) const {
    if (!bloom_bits) return true;
    uint64_t h = hash64(key.data(), key.size(), 0), delta = (h >> 17) | (h << 47);
    for (int k = 0; k < 7; ++k) {
      uint64_t b = h % bloom_bits;
      if (!(bloom[b >> 3] & (1 << (b & 7)))) { bloom_skips.fetch_add(1, std::memory_order_relaxed); return false; }
      h += delta;
    }
    return true;
  }

  // The checksum of a block is computed on its first use; the mapping is read-only, so once is enough.
  bool check_block(size_t b) const {
    if (verified[b].load(std::memory_order_acquire)) return true;
    const BlockHandle& h = index[b];
    if (crc32(map + h.offset, h.bytes) != get_fixed<uint32_t>(map + h.offset + h.bytes)) return false;
    verified[b].store(1, std::memory_order_release);
    return true;
  }

  // Point lookup: 1 put, 2 delete, 0 absent, -1 damaged.  Walks the one block that can hold the key.
  int find(const Bytes& key, Bytes* out, std::string* err) const {
    size_t b = block_for(key);
    if (b >= index.size()) return 0;
    if (!check_block(b)) { *err = path + ": data block checksum"; return -1; }
    const uint8_t *p = map + index[b].offset, *end = p + index[b].bytes;
    while (p < end) {
      uint8_t kind = *p;
      uint64_t kl, vl;
      const uint8_t* q = get_varint(p + 1, end, &kl);
      if (q) q = get_varint(q, end, &vl);
      if (!q || kl > uint64_t(end - q) || vl > uint64_t(end - q) - kl) { *err = path + ": entry runs off its block"; return -1; }
      int c = compare(q, kl, key);
      if (c == 0) {
        if (kind == kPut && out) out->assign(reinterpret_cast<const char*>(q + kl), vl);
        return kind == kPut ? 1 : 2;
      }
      if (c > 0) return 0;
      p = q + kl + vl;
    }
    return 0;
  }

  // Offsets of the entries of block b (relative to the block); verifies the block's checksum and framing.
  std::string parse_block(size_t b, std::vector<uint32_t>* offs) const {
    const BlockHandle& h = index[b];
    const uint8_t *base = map + h.offset, *p = base, *end = base + h.bytes;
    if (!check_block(b)) return path + ": data block checksum";
    offs->clear();
    while (p < end) {
      offs->push_back(uint32_t(p - base));
      uint64_t kl, vl;
      const uint8_t* q = get_varint(p + 1, end, &kl);
      if (q) q = get_varint(q, end, &vl);
      if (!q || kl > uint64_t(end - q) || vl > uint64_t(end - q) - kl) return path + ": entry runs off its block";
      p = q + kl + vl;
    }
    return "";
  }

  Entry entry_at(size_t b, uint32_t off) const {                       // off comes from parse_block
    const uint8_t *base = map + index[b].offset, *end = base + index[b].bytes, *p = base + off;
    Entry e;
    e.kind = *p;
    uint64_t kl = 0, vl = 0;
    const uint8_t* q = get_varint(p + 1, end, &kl);
    q = get_varint(q, end, &vl);
    e.key = q; e.klen = uint32_t(kl); e.val = q + kl; e.vlen = uint32_t(vl);
    return e;
  }

  // First block whose last key is >= key (index.size() when every key is smaller).
  size_t block_for(const Bytes& key) const {
    size_t lo = 0, hi = index.size();
    while (lo < hi) {
      size_t mid = (lo + hi) / 2;
      if (index[mid].last_key < key) lo = mid + 1; else hi = mid;
    }
    return lo;
  }
};


// ---- memory tables ------------------------------------------------------------------------------------------
struct MemVersion { uint64_t seq; uint8_t kind; Bytes value; };

// Ordered rows, each with its versions newest first.  Rows are never erased (a delete is a version), so a reader
// that re-finds its position by key under the shared lock is never left dangling.
struct MemTable {
  std::map<Bytes, std::vector<MemVersion>> rows;
  mutable std::shared_mutex mu;
  std::atomic<size_t> bytes{0};
  uint64_t wal_number = 0;

  // min_snapshot: the oldest sequence number some reader still looks at (UINT64_MAX: nobody).
  void apply(const Bytes& key, uint8_t kind, const Bytes& value, uint64_t seq, uint64_t min_snapshot) {
    auto& v = rows[key];
    if (v.empty()) bytes += key.size() + 48;
    if (min_snapshot == UINT64_MAX) {
      for (auto& old : v) bytes -= old.value.size() + 24;
      v.clear();
    } else {
      // keep the newest version a reader at min_snapshot sees, and everything newer
      size_t keep = v.size();
      for (size_t i = 0; i < v.size(); ++i) if (v[i].seq <= min_snapshot) { keep = i + 1; break; }
      for (size_t i = keep; i < v.size(); ++i) bytes -= v[i].value.size() + 24;
      v.resize(keep);
    }
    v.insert(v.begin(), MemVersion{seq, kind, value});
    bytes += value.size() + 24;
  }
  static const MemVersion* visible(const std::vector<MemVersion>& v, uint64_t seq) {
    for (auto& m : v) if (m.seq <= seq) return &m;
    return nullptr;
  }
  // 1 found (put), 2 found (delete), 0 no version visible
  int get(const Bytes& key, uint64_t seq, Bytes* out) const {
    std::shared_lock<std::shared_mutex> l(mu);
    auto it = rows.find(key);
    if (it == rows.end()) return 0;
    const MemVersion* m = visible(it->second, seq);
    if (!m) return 0;
    if (m->kind == kPut && out) *out = m->value;
    return m->kind;
  }
};

// ---- ordered sources and their merge ------------------------------------------------------------------------
struct Source {
  bool valid = false;
  Bytes key;
  const uint8_t* val = nullptr;
  size_t vlen = 0;
  uint8_t kind = 0;
  std::string error;
  virtual ~Source() {}
  virtual void seek_ge(const Bytes& k) = 0;
  virtual void seek_le(const Bytes& k) = 0;
  virtual void next() = 0;
  virtual void prev() = 0;
};

struct MemSource : Source {
  std::shared_ptr<MemTable> t;
  uint64_t seq;
  Bytes owned;
  MemSource(std::shared_ptr<MemTable> m, uint64_t s) : t(std::move(m)), seq(s) {}
  using It = std::map<Bytes, std::vector<MemVersion>>::const_iterator;
  void load(It it, bool forward) {
    // skips rows with no version this reader may see
    for (;;) {
      if (it == t->rows.end()) { valid = false; return; }
      if (const MemVersion* m = MemTable::visible(it->second, seq)) {
        valid = true; key = it->first; kind = m->kind; owned = m->value;
        val = reinterpret_cast<const uint8_t*>(owned.data()); vlen = owned.size();
        return;
      }
      if (forward) ++it;
      else { if (it == t->rows.begin()) { valid = false; return; } --it; }
    }
  }
  void seek_ge(const Bytes& k) override {
    std::shared_lock<std::shared_mutex> l(t->mu);
    load(t->rows.lower_bound(k), true);
  }
  void seek_le(const Bytes& k) override {
    std::shared_lock<std::shared_mutex> l(t->mu);
    auto it = t->rows.upper_bound(k);
    if (it == t->rows.begin()) { valid = false; return; }
    load(--it, false);
  }
  void next() override {
    std::shared_lock<std::shared_mutex> l(t->mu);
    load(t->rows.upper_bound(key), true);
  }
  void prev() override {
    std::shared_lock<std::shared_mutex> l(t->mu);
    auto it = t->rows.lower_bound(key);
    if (it == t->rows.begin()) { valid = false; return; }
    load(--it, false);
  }
};

struct TableSource : Source {
  std::shared_ptr<Table> t;
  size_t block = 0, pos = 0;
  std::vector<uint32_t> offs;
  explicit TableSource(std::shared_ptr<Table> tb) : t(std::move(tb)) {}
  bool open_block(size_t b) {
    block = b;
    std::string e = t->parse_block(b, &offs);
    if (!e.empty()) { error = e; valid = false; return false; }
    return true;
  }
  void load() {
    Entry e = t->entry_at(block, offs[pos]);
    valid = true; kind = e.kind;
    key.assign(reinterpret_cast<const char*>(e.key), e.klen);
    val = e.val; vlen = e.vlen;
  }
  size_t lower(const Bytes& k) const {                                  // first entry of the open block >= k
    size_t lo = 0, hi = offs.size();
    while (lo < hi) {
      size_t mid = (lo + hi) / 2;
      Entry e = t->entry_at(block, offs[mid]);
      if (compare(e.key, e.klen, k) < 0) lo = mid + 1; else hi = mid;
    }
    return lo;
  }
  void first() { if (t->index.empty() || !open_block(0) || offs.empty()) { valid = false; return; } pos = 0; load(); }
  void last() {
    if (t->index.empty() || !open_block(t->index.size() - 1) || offs.empty()) { valid = false; return; }
    pos = offs.size() - 1; load();
  }
  void seek_ge(const Bytes& k) override {
    size_t b = t->block_for(k);
    if (b >= t->index.size() || !open_block(b)) { valid = false; return; }
    pos = lower(k);
    if (pos >= offs.size()) { valid = false; return; }
    load();
  }
  void seek_le(const Bytes& k) override {
    size_t b = t->block_for(k);
    if (b >= t->index.size()) { last(); return; }
    if (!open_block(b)) return;
    pos = lower(k);
    if (pos < offs.size()) {
      Entry e = t->entry_at(block, offs[pos]);
      if (compare(e.key, e.klen, k) == 0) { load(); return; }
    }
    step_back();
  }
  void step_back() {
    if (pos > 0) { --pos; load(); return; }
    if (block == 0) { valid = false; return; }
    if (!open_block(block - 1) || offs.empty()) { valid = false; return; }
    pos = offs.size() - 1; load();
  }
  void next() override {
    if (!valid) return;
    if (pos + 1 < offs.size()) { ++pos; load(); return; }
    if (block + 1 >= t->index.size() || !open_block(block + 1) || offs.empty()) { valid = false; return; }
    pos = 0; load();
  }
  void prev() override { if (valid) step_back(); }
};

// The files of one level below level 0: disjoint key ranges in ascending order, read as one run.
struct LevelSource : Source {
  std::vector<std::shared_ptr<Table>> files;
  std::unique_ptr<TableSource> cur;
  size_t at = 0;
  explicit LevelSource(std::vector<std::shared_ptr<Table>> f) : files(std::move(f)) {}
  void adopt() {
    valid = cur && cur->valid;
    if (cur && !cur->error.empty()) error = cur->error;
    if (valid) { key = cur->key; val = cur->val; vlen = cur->vlen; kind = cur->kind; }
  }
  void open(size_t i) { at = i; cur.reset(new TableSource(files[i])); }
  void seek_ge(const Bytes& k) override {
    size_t lo = 0, hi = files.size();
    while (lo < hi) { size_t mid = (lo + hi) / 2; if (files[mid]->largest < k) lo = mid + 1; else hi = mid; }
    if (lo >= files.size()) { valid = false; return; }
    open(lo); cur->seek_ge(k); adopt();
  }
  void seek_le(const Bytes& k) override {
    size_t lo = 0, hi = files.size();                                   // first file whose smallest key is > k
    while (lo < hi) { size_t mid = (lo + hi) / 2; if (files[mid]->smallest <= k) lo = mid + 1; else hi = mid; }
    if (lo == 0) { valid = false; return; }
    open(lo - 1); cur->seek_le(k); adopt();
  }
  void next() override {
    if (!valid) return;
    cur->next();
    if (!cur->valid && cur->error.empty() && at + 1 < files.size()) { open(at + 1); cur->first(); }
    adopt();
  }
  void prev() override {
    if (!valid) return;
    cur->prev();
    if (!cur->valid && cur->error.empty() && at > 0) { open(at - 1); cur->last(); }
    adopt();
  }
};

// Newest source first: among equal keys the lowest index wins, and a winning delete hides the key.
struct Merged {
  std::vector<std::unique_ptr<Source>> src;
  int direction = 0;                                                     // +1 forward, -1 backward
  bool valid = false;
  Bytes key;
  const uint8_t* val = nullptr;
  size_t vlen = 0;
  uint8_t kind = 0;                                                      // kind of the winner (raw mode only)
  bool raw = false;                                                      // raw: deletes are returned, not hidden
  std::string error;

  bool failed() {
    for (auto& s : src) if (!s->error.empty()) { error = s->error; valid = false; return true; }
    return false;
  }
  void settle() {
    for (;;) {
      if (failed()) return;
      Source* best = nullptr;
      for (auto& s : src) {
        if (!s->valid) continue;
        if (!best) { best = s.get(); continue; }
        int c = s->key.compare(best->key);
        if (direction > 0 ? c < 0 : c > 0) best = s.get();
      }
      if (!best) { valid = false; return; }
      key = best->key; val = best->val; vlen = best->vlen; kind = best->kind; valid = true;
      if (best->kind != kDel || raw) return;
      step_equal();
    }
  }
  void step_equal() {                                                    // moves every source off the current key
    for (auto& s : src)
      if (s->valid && s->key == key) { if (direction > 0) s->next(); else s->prev(); }
  }
  void seek_ge(const Bytes& k) { direction = 1; for (auto& s : src) s->seek_ge(k); settle(); }
  void seek_le(const Bytes& k) { direction = -1; for (auto& s : src) s->seek_le(k); settle(); }
  void next() {
    if (!valid) return;
    if (direction < 0) {
      direction = 1;
      for (auto& s : src) { s->seek_ge(key); }
    }
    Bytes k = key;
    for (auto& s : src) if (s->valid && s->key == k) s->next();
    settle();
  }
  void prev() {
    if (!valid) return;
    if (direction > 0) {
      direction = -1;
      for (auto& s : src) { s->seek_le(key); }
    }
    Bytes k = key;
    for (auto& s : src) if (s->valid && s->key == k) s->prev();
    settle();
  }
};

// ---- versions -----------------------------------------------------------------------------------------------
struct Version {
  std::shared_ptr<MemTable> mem;
  std::vector<std::shared_ptr<MemTable>> imm;                           // newest first
  std::vector<std::shared_ptr<Table>> levels[kLevels];                  // level 0 newest first; others by key

  void sources(uint64_t seq, std::vector<std::unique_ptr<Source>>* out) const {
    out->emplace_back(new MemSource(mem, seq));
    for (auto& m : imm) out->emplace_back(new MemSource(m, seq));
    for (auto& t : levels[0]) out->emplace_back(new TableSource(t));
    for (int l = 1; l < kLevels; ++l)
      if (!levels[l].empty()) out->emplace_back(new LevelSource(levels[l]));
  }

  // 1 found, 0 absent or deleted, -1 a damaged file (message in *err)
  int get(const Bytes& key, uint64_t seq, Bytes* out, std::string* err) const {
    int r = mem->get(key, seq, out);
    if (r) return r == kPut;
    for (auto& m : imm) if ((r = m->get(key, seq, out))) return r == kPut;
    auto in_table = [&](const std::shared_ptr<Table>& t) -> int {      // 1 put, 2 delete, 0 absent, -1 damaged
      if (key < t->smallest || key > t->largest || !t->may_contain(key)) return 0;
      return t->find(key, out, err);
    };
    for (auto& t : levels[0]) if ((r = in_table(t))) return r < 0 ? -1 : r == kPut;
    for (int l = 1; l < kLevels; ++l) {
      auto& f = levels[l];
      size_t lo = 0, hi = f.size();
      while (lo < hi) { size_t mid = (lo + hi) / 2; if (f[mid]->largest < key) lo = mid + 1; else hi = mid; }
      if (lo < f.size() && (r = in_table(f[lo]))) return r < 0 ? -1 : r == kPut;
    }
    return 0;
  }
};

// ---- the store ----------------------------------------------------------------------------------------------
struct Options {
  uint64_t memtable_bytes = 8ull << 20;
  uint64_t block_bytes = 16 << 10;
  uint64_t target_file_bytes = 32ull << 20;
  uint64_t level1_bytes = 64ull << 20;                                  // each deeper level holds ten times more
  int l0_compact = 4, l0_stall = 12;
  int sync = 1;                                                          // 0: leave it to the OS, 1: every commit
  int read_only = 0;
  int background = 1;                                                    // 0: flush / compact only when asked
};

struct Op { uint8_t kind; Bytes key, value; };

bool parse_ops(const uint8_t* p, size_t n, std::vector<Op>* ops) {
  const uint8_t* end = p + n;
  while (p < end) {
    Op op;
    op.kind = *p++;
    uint64_t kl, vl;
    if (op.kind != kPut && op.kind != kDel) return false;
    p = get_varint(p, end, &kl);
    if (p) p = get_varint(p, end, &vl);
    if (!p || kl > uint64_t(end - p) || vl > uint64_t(end - p) - kl) return false;
    op.key.assign(reinterpret_cast<const char*>(p), kl);
    op.value.assign(reinterpret_cast<const char*>(p + kl), vl);
    p += kl + vl;
    ops->push_back(std::move(op));
  }
  return true;
}

struct Stats {
  uint64_t mutable_bytes, immutable_bytes, immutable_tables, level_files[kLevels], level_bytes[kLevels], flushes,
      compactions, compaction_bytes_read, compaction_bytes_written, wal_bytes, wal_records, stalls, stall_ms,
      bloom_skips, last_sequence, live_snapshots, ingests, recovered_records, dropped_tombstones;
};

struct Store {
  std::string dir;
  Options opt;
  int lock_fd = -1, wal_fd = -1;
  std::mutex mu;                         // current version, queues, counters
  std::mutex write_mu;                   // one commit at a time
  std::mutex manifest_mu;                // one publisher at a time; taken before mu
  std::mutex snap_mu;                    // live snapshot set against memtable trimming
  std::condition_variable work_cv, done_cv;
  std::shared_ptr<const Version> current;
  std::multiset<uint64_t> snapshots;
  std::atomic<uint64_t> last_seq{0};
  uint64_t next_file = 1, wal_number = 0;
  size_t compact_pointer[kLevels] = {0};
  bool stopping = false;
  std::mutex compact_mu;                 // one merge at a time, whoever runs it
  std::string bg_error;
  std::thread flush_thread, compact_thread;
  Stats st{};

  std::string table_path(uint64_t n) const { return dir + "/" + std::to_string(n) + ".tbl"; }
  std::string wal_path(uint64_t n) const { return dir + "/wal-" + std::to_string(n) + ".log"; }

  // ---- manifest ----
  bool write_manifest(const Version& v, uint64_t min_wal, uint64_t next_number, std::string* err) {
    std::string body;
    for (int l = 0; l < kLevels; ++l)
      for (auto& t : v.levels[l])
        body += "file " + std::to_string(l) + " " + std::to_string(t->number) + " " + std::to_string(t->bytes) + " " +
                std::to_string(t->entries) + " " + hex(t->smallest) + " " + hex(t->largest) + "\n";
    body += "next " + std::to_string(next_number) + "\nseq " + std::to_string(last_seq.load()) + "\nwal " +
            std::to_string(min_wal) + "\n";
    body += "crc " + std::to_string(crc32(reinterpret_cast<const uint8_t*>(body.data()), body.size())) + "\n";
    std::string tmp = dir + "/MANIFEST.tmp";
    int fd = ::open(tmp.c_str(), O_CREAT | O_TRUNC | O_WRONLY, 0644);
    if (fd < 0 || !write_all(fd, body.data(), body.size()) || ::fsync(fd) != 0) {
      if (fd >= 0) ::close(fd);
      *err = "cannot write " + tmp;
      return false;
    }
    ::close(fd);
    if (::rename(tmp.c_str(), (dir + "/MANIFEST").c_str()) != 0) { *err = "cannot replace MANIFEST"; return false; }
    sync_dir(dir);
    return true;
  }

  uint64_t oldest_needed_wal(const Version& v) const {
    uint64_t n = v.mem->wal_number;
    for (auto& m : v.imm) n = std::min(n, m->wal_number);
    return n;
  }

  void remove_wals_below(uint64_t n) {
    DIR* d = ::opendir(dir.c_str());
    if (!d) return;
    while (dirent* e = ::readdir(d)) {
      unsigned long long w;
      if (std::sscanf(e->d_name, "wal-%llu.log", &w) == 1 && w < n) ::unlink((dir + "/" + e->d_name).c_str());
    }
    ::closedir(d);
  }

  // ---- write-ahead log ----
  bool open_wal(uint64_t n, std::string* err) {
    if (wal_fd >= 0) ::close(wal_fd);
    wal_fd = ::open(wal_path(n).c_str(), O_CREAT | O_WRONLY | O_APPEND, 0644);
    if (wal_fd < 0) { *err = "cannot create " + wal_path(n); return false; }
    wal_number = n;
    return true;
  }

  // Replays one log into t; stops at the first record that is cut short or fails its checksum (a torn tail).
  void replay_wal(const std::string& path, MemTable* t) {
    int fd = ::open(path.c_str(), O_RDONLY);
    if (fd < 0) return;
    struct stat s;
    if (::fstat(fd, &s) != 0 || s.st_size == 0) { ::close(fd); return; }
    void* m = ::mmap(nullptr, size_t(s.st_size), PROT_READ, MAP_SHARED, fd, 0);
    ::close(fd);
    if (m == MAP_FAILED) return;
    const uint8_t *p = static_cast<const uint8_t*>(m), *end = p + s.st_size;
    while (end - p >= 8) {
      uint32_t n = get_fixed<uint32_t>(p), c = get_fixed<uint32_t>(p + 4);
      if (n < 8 || n > uint64_t(end - p - 8) || crc32(p + 8, n) != c) break;
      uint64_t seq = get_fixed<uint64_t>(p + 8);
      std::vector<Op> ops;
      if (!parse_ops(p + 16, n - 8, &ops)) break;
      for (auto& op : ops) t->apply(op.key, op.kind, op.value, seq++, UINT64_MAX);
      if (seq - 1 > last_seq.load()) last_seq.store(seq - 1);
      ++st.recovered_records;
      p += 8 + n;
    }
    ::munmap(m, size_t(s.st_size));
  }

  // ---- open ----
  std::string open(const std::string& d, const Options& o) {
    dir = d; opt = o;
    if (!opt.read_only) {
      ::mkdir(dir.c_str(), 0755);
      lock_fd = ::open((dir + "/LOCK").c_str(), O_CREAT | O_RDWR, 0644);
      if (lock_fd < 0 || ::flock(lock_fd, LOCK_EX | LOCK_NB) != 0)
        return dir + ": another process holds the store open for writing";
    }
    auto v = std::make_shared<Version>();
    v->mem = std::make_shared<MemTable>();
    uint64_t min_wal = 0;
    std::set<uint64_t> live;
    if (FILE* f = std::fopen((dir + "/MANIFEST").c_str(), "r")) {
      std::string body, all;
      char line[8192];
      bool crc_ok = false;
      std::vector<std::string> lines;
      while (std::fgets(line, sizeof line, f)) lines.emplace_back(line);
      std::fclose(f);
      for (auto& ln : lines) {
        unsigned long long c;
        if (std::sscanf(ln.c_str(), "crc %llu", &c) == 1) {
          crc_ok = crc32(reinterpret_cast<const uint8_t*>(body.data()), body.size()) == uint32_t(c);
          break;
        }
        body += ln;
      }
      if (!crc_ok) return dir + "/MANIFEST: checksum does not match";
      for (auto& ln : lines) {
        int level; unsigned long long num, bytes, entries, x;
        char lo[4100], hi[4100];
        if (std::sscanf(ln.c_str(), "file %d %llu %llu %llu %4099s %4099s", &level, &num, &bytes, &entries, lo, hi) == 6) {
          if (level < 0 || level >= kLevels) return dir + "/MANIFEST: level out of range";
          auto t = std::make_shared<Table>();
          std::string e = t->open(table_path(num));
          if (!e.empty()) return e;
          if (t->bytes != bytes || t->entries != entries) return t->path + ": size or entry count differs from the manifest";
          t->number = num; t->level = level; t->smallest = unhex(lo); t->largest = unhex(hi);
          v->levels[level].push_back(t);
          live.insert(num);
        } else if (std::sscanf(ln.c_str(), "next %llu", &x) == 1) next_file = x;
        else if (std::sscanf(ln.c_str(), "seq %llu", &x) == 1) last_seq.store(x);
        else if (std::sscanf(ln.c_str(), "wal %llu", &x) == 1) min_wal = x;
      }
      std::sort(v->levels[0].begin(), v->levels[0].end(), [](auto& a, auto& b) { return a->number > b->number; });
      for (int l = 1; l < kLevels; ++l)
        std::sort(v->levels[l].begin(), v->levels[l].end(), [](auto& a, auto& b) { return a->smallest < b->smallest; });
    } else if (opt.read_only) {
      return dir + ": no MANIFEST (not a store directory)";
    }
    // logs at or above the manifest's mark, oldest first; table files the manifest does not name are leftovers
    std::vector<uint64_t> wals;
    if (DIR* dd = ::opendir(dir.c_str())) {
      while (dirent* e = ::readdir(dd)) {
        unsigned long long n;
        char tail[8];
        if (std::sscanf(e->d_name, "wal-%llu.lo%1s", &n, tail) == 2) { if (n >= min_wal) wals.push_back(n); }
        else if (std::sscanf(e->d_name, "%llu.tb%1s", &n, tail) == 2) {
          if (!live.count(n) && !opt.read_only) ::unlink((dir + "/" + e->d_name).c_str());
          next_file = std::max<uint64_t>(next_file, n + 1);
        }
      }
      ::closedir(dd);
    }
    std::sort(wals.begin(), wals.end());
    for (uint64_t w : wals) { replay_wal(wal_path(w), v->mem.get()); next_file = std::max(next_file, w + 1); }
    current = v;
    if (opt.read_only) return "";
    std::string err;
    uint64_t fresh = next_file++;
    if (v->mem->bytes.load() > 0) {
      // what the logs held goes to a table file at once, so the old logs can go
      std::shared_ptr<Table> t;
      if (!build_from_mem(*v->mem, &t, &err)) return err;
      auto nv = std::make_shared<Version>(*v);
      nv->mem = std::make_shared<MemTable>();
      if (t) nv->levels[0].insert(nv->levels[0].begin(), t);
      current = v = nv;
    }
    v->mem->wal_number = fresh;
    if (!open_wal(fresh, &err)) return err;
    if (!write_manifest(*v, fresh, next_file, &err)) return err;
    remove_wals_below(fresh);
    if (opt.background) {
      flush_thread = std::thread([this] { flush_loop(); });
      compact_thread = std::thread([this] { compact_loop(); });
    }
    return "";
  }

  // The newest version of every row of a memory table as one level-0 table file (deletes included).
  bool build_from_mem(const MemTable& m, std::shared_ptr<Table>* out, std::string* err) {
    uint64_t num;
    { std::lock_guard<std::mutex> l(mu); num = next_file++; }
    TableBuilder b(table_path(num), opt.block_bytes);
    {
      std::shared_lock<std::shared_mutex> l(m.mu);
      for (auto& row : m.rows) if (!row.second.empty()) b.add(row.first, row.second[0].kind, row.second[0].value);
    }
    if (b.entries == 0) { b.finish(false); ::unlink(b.path.c_str()); out->reset(); return true; }
    if (!b.finish(opt.sync != 0)) { *err = "cannot write " + b.path; return false; }
    auto t = std::make_shared<Table>();
    std::string e = t->open(b.path);
    if (!e.empty()) { *err = e; return false; }
    t->number = num; t->level = 0;
    *out = t;
    return true;
  }

  // ---- publishing a new version ----
  // Removes the tables numbered in `gone`, adds `add` at their levels, drops the immutable table `flushed` (if
  // any), then persists the manifest.  Old logs and replaced files go once the manifest names their successors.
  bool publish(const std::set<uint64_t>& gone, const std::vector<std::shared_ptr<Table>>& add, const MemTable* flushed,
               std::string* err) {
    std::lock_guard<std::mutex> pm(manifest_mu);
    std::shared_ptr<const Version> old;
    std::shared_ptr<Version> nv;
    uint64_t next_number;
    {
      std::lock_guard<std::mutex> l(mu);
      old = current;
      nv = std::make_shared<Version>(*old);
      if (flushed)
        nv->imm.erase(std::remove_if(nv->imm.begin(), nv->imm.end(), [&](auto& m) { return m.get() == flushed; }),
                      nv->imm.end());
      for (int lv = 0; lv < kLevels; ++lv) {
        auto& f = nv->levels[lv];
        f.erase(std::remove_if(f.begin(), f.end(), [&](auto& t) { return gone.count(t->number) > 0; }), f.end());
      }
      for (auto& t : add) nv->levels[t->level].push_back(t);
      std::sort(nv->levels[0].begin(), nv->levels[0].end(), [](auto& a, auto& b) { return a->number > b->number; });
      for (int lv = 1; lv < kLevels; ++lv)
        std::sort(nv->levels[lv].begin(), nv->levels[lv].end(), [](auto& a, auto& b) { return a->smallest < b->smallest; });
      current = nv;
      next_number = next_file;
    }
    uint64_t min_wal = oldest_needed_wal(*nv);
    if (!write_manifest(*nv, min_wal, next_number, err)) return false;
    for (int lv = 0; lv < kLevels; ++lv)
      for (auto& t : old->levels[lv]) if (gone.count(t->number)) t->obsolete.store(true);
    remove_wals_below(min_wal);
    return true;
  }

  // ---- commits ----
  int write(const uint8_t* payload, size_t n, std::string* err) {
    if (opt.read_only) { *err = "the store is open read-only"; return -1; }
    std::vector<Op> ops;
    if (!parse_ops(payload, n, &ops)) { *err = "malformed batch"; return -1; }
    for (auto& op : ops) if (op.key.empty() || op.key.size() > 1024) { *err = "keys are 1 to 1024 bytes"; return -1; }
    if (ops.empty()) return 0;
    std::lock_guard<std::mutex> w(write_mu);
    if (!wait_for_room(err)) return -1;
    uint64_t first = last_seq.load() + 1;
    Bytes rec;
    put_fixed<uint32_t>(rec, uint32_t(n + 8));
    put_fixed<uint32_t>(rec, 0);
    put_fixed<uint64_t>(rec, first);
    rec.append(reinterpret_cast<const char*>(payload), n);
    uint32_t c = crc32(reinterpret_cast<const uint8_t*>(rec.data()) + 8, n + 8);
    std::memcpy(&rec[4], &c, 4);
    if (!write_all(wal_fd, rec.data(), rec.size()) || (opt.sync && ::fdatasync(wal_fd) != 0)) {
      *err = "cannot append to the write-ahead log";
      return -1;
    }
    std::shared_ptr<MemTable> mem;
    { std::lock_guard<std::mutex> l(mu); mem = current->mem; st.wal_bytes += rec.size(); ++st.wal_records; }
    {
      std::lock_guard<std::mutex> s(snap_mu);
      uint64_t min_snap = snapshots.empty() ? UINT64_MAX : *snapshots.begin();
      std::unique_lock<std::shared_mutex> ml(mem->mu);
      uint64_t seq = first;
      for (auto& op : ops) mem->apply(op.key, op.kind, op.value, seq++, min_snap);
      last_seq.store(seq - 1);
    }
    if (mem->bytes.load() >= opt.memtable_bytes) return rotate(err) ? 0 : -1;
    return 0;
  }

  // Caller holds write_mu.  The full table joins the immutable queue; commits continue into a fresh one and log.
  bool rotate(std::string* err) {
    uint64_t n;
    { std::lock_guard<std::mutex> l(mu); if (current->mem->bytes.load() == 0) return true; n = next_file++; }
    if (!open_wal(n, err)) return false;
    {
      std::lock_guard<std::mutex> l(mu);
      auto nv = std::make_shared<Version>(*current);
      nv->imm.insert(nv->imm.begin(), nv->mem);
      nv->mem = std::make_shared<MemTable>();
      nv->mem->wal_number = n;
      current = nv;
    }
    work_cv.notify_all();
    return true;
  }

  // Caller holds write_mu.  Hard pressure delays the commit for a bounded time; with no background threads the
  // writer does the work itself.
  bool wait_for_room(std::string* err) {
    std::unique_lock<std::mutex> l(mu);
    auto crowded = [&] { return current->imm.size() >= 2 || int(current->levels[0].size()) >= opt.l0_stall; };
    if (!crowded()) return true;
    ++st.stalls;
    auto t0 = std::chrono::steady_clock::now();
    if (!opt.background) {
      l.unlock();
      bool ok = drain(err);
      l.lock();
      return ok;
    }
    work_cv.notify_all();
    bool ok = done_cv.wait_for(l, std::chrono::seconds(60), [&] { return !crowded() || !bg_error.empty(); });
    st.stall_ms += uint64_t(std::chrono::duration_cast<std::chrono::milliseconds>(
                                std::chrono::steady_clock::now() - t0).count());
    if (!bg_error.empty()) { *err = "background work failed: " + bg_error; return false; }
    if (!ok) { *err = "write stalled for 60 s waiting for flushes and compactions"; return false; }
    return true;
  }

  // ---- flush ----
  bool flush_one(std::string* err) {                                     // false: nothing to do or failed
    std::shared_ptr<MemTable> m;
    { std::lock_guard<std::mutex> l(mu); if (current->imm.empty()) return false; m = current->imm.back(); }
    std::shared_ptr<Table> t;
    if (!build_from_mem(*m, &t, err)) return false;
    std::vector<std::shared_ptr<Table>> add;
    if (t) add.push_back(t);
    if (!publish({}, add, m.get(), err)) return false;
    { std::lock_guard<std::mutex> l(mu); ++st.flushes; }
    done_cv.notify_all();
    return true;
  }

  // ---- compaction ----
  uint64_t level_target(int l) const {
    uint64_t t = opt.level1_bytes;
    for (int i = 1; i < l; ++i) t *= 10;
    return t;
  }

  // Picks the level most over its budget.  Returns the inputs (newest first) and the output level, or -1.
  int pick(std::vector<std::shared_ptr<Table>>* inputs, bool force_all) {
    std::lock_guard<std::mutex> l(mu);
    const Version& v = *current;
    if (force_all) {                                                     // everything into the deepest level in use
      int deepest = 1;
      size_t files = 0;
      for (int lv = 0; lv < kLevels; ++lv) { if (!v.levels[lv].empty() && lv > deepest) deepest = lv; files += v.levels[lv].size(); }
      if (files == 0 || (files == 1 && v.levels[0].empty())) return -1;
      for (int lv = 0; lv <= deepest; ++lv) for (auto& t : v.levels[lv]) inputs->push_back(t);
      return deepest;
    }
    double best = 0;
    int from = -1;
    for (int lv = 0; lv + 1 < kLevels; ++lv) {
      double score;
      if (lv == 0) score = double(v.levels[0].size()) / opt.l0_compact;
      else {
        uint64_t b = 0;
        for (auto& t : v.levels[lv]) b += t->bytes;
        score = double(b) / double(level_target(lv));
      }
      if (score >= 1.0 && score > best) { best = score; from = lv; }
    }
    if (from < 0) return -1;
    Bytes lo, hi;
    if (from == 0) {
      for (auto& t : v.levels[0]) {
        if (inputs->empty() || t->smallest < lo) lo = t->smallest;
        if (inputs->empty() || t->largest > hi) hi = t->largest;
        inputs->push_back(t);
      }
    } else {
      auto& f = v.levels[from];
      auto& t = f[compact_pointer[from]++ % f.size()];
      lo = t->smallest; hi = t->largest;
      inputs->push_back(t);
    }
    for (auto& t : v.levels[from + 1]) if (!(t->largest < lo || t->smallest > hi)) inputs->push_back(t);
    return from + 1;
  }

  bool compact_one(bool force_all, std::string* err) {                   // false: nothing to do or failed
    std::lock_guard<std::mutex> only(compact_mu);
    std::vector<std::shared_ptr<Table>> inputs;
    int out_level = pick(&inputs, force_all);
    if (out_level < 0) return false;
    bool bottom;
    {
      std::lock_guard<std::mutex> l(mu);
      bottom = true;
      for (int lv = out_level + 1; lv < kLevels; ++lv) if (!current->levels[lv].empty()) bottom = false;
    }
    Merged m;
    m.raw = true;
    // level-0 inputs are listed newest first; everything deeper is older than them and disjoint within its level
    for (auto& t : inputs) m.src.emplace_back(new TableSource(t));
    std::stable_sort(m.src.begin(), m.src.end(), [](auto& a, auto& b) {
      auto *x = static_cast<TableSource*>(a.get()), *y = static_cast<TableSource*>(b.get());
      if (x->t->level != y->t->level) return x->t->level < y->t->level;
      return x->t->level == 0 && x->t->number > y->t->number;
    });
    std::vector<std::shared_ptr<Table>> outputs;
    std::unique_ptr<TableBuilder> b;
    uint64_t num = 0, read = 0, written = 0, dropped = 0;
    auto close_output = [&]() -> bool {
      if (!b) return true;
      uint64_t bytes = b->finish(opt.sync != 0);
      if (!bytes) { *err = "cannot write " + b->path; return false; }
      auto t = std::make_shared<Table>();
      std::string e = t->open(b->path);
      if (!e.empty()) { *err = e; return false; }
      t->number = num; t->level = out_level;
      outputs.push_back(t);
      written += bytes;
      b.reset();
      return true;
    };
    bool ok = true;
    m.seek_ge(Bytes());
    for (; m.valid; m.next()) {
      if (m.kind == kDel && bottom) { ++dropped; continue; }
      if (!b) {
        { std::lock_guard<std::mutex> l(mu); num = next_file++; }
        b.reset(new TableBuilder(table_path(num), opt.block_bytes));
      }
      b->add(m.key, m.kind, Bytes(reinterpret_cast<const char*>(m.val), m.vlen));
      if (b->offset + b->block.size() >= opt.target_file_bytes && !(ok = close_output())) break;
    }
    if (ok && !m.error.empty()) { *err = m.error; ok = false; }
    ok = ok && close_output();
    std::set<uint64_t> gone;
    for (auto& t : inputs) { gone.insert(t->number); read += t->bytes; }
    if (ok) ok = publish(gone, outputs, nullptr, err);
    if (!ok) { for (auto& t : outputs) t->obsolete.store(true); return false; }
    {
      std::lock_guard<std::mutex> l(mu);
      ++st.compactions; st.compaction_bytes_read += read; st.compaction_bytes_written += written;
      st.dropped_tombstones += dropped;
    }
    done_cv.notify_all();
    return true;
  }

  // Flushes every immutable table and compacts until no level is over budget (the caller's thread does the work).
  bool drain(std::string* err) {
    for (;;) {
      std::string e;
      if (flush_one(&e)) continue;
      if (!e.empty()) { *err = e; return false; }
      if (compact_one(false, &e)) continue;
      if (!e.empty()) { *err = e; return false; }
      return true;
    }
  }

  void flush_loop() {
    std::unique_lock<std::mutex> l(mu);
    while (!stopping) {
      if (current->imm.empty() || !bg_error.empty()) { work_cv.wait_for(l, std::chrono::milliseconds(200)); continue; }
      l.unlock();
      std::string e;
      bool did = flush_one(&e);
      l.lock();
      if (!did && !e.empty()) bg_error = e;
      done_cv.notify_all();
      work_cv.notify_all();
    }
  }

  void compact_loop() {
    std::unique_lock<std::mutex> l(mu);
    while (!stopping) {
      if (!bg_error.empty()) { work_cv.wait_for(l, std::chrono::milliseconds(200)); continue; }
      l.unlock();
      std::string e;
      bool did = compact_one(false, &e);
      l.lock();
      if (!did && !e.empty()) bg_error = e;
      done_cv.notify_all();
      if (!did && !stopping) work_cv.wait_for(l, std::chrono::milliseconds(200));
    }
  }

  // Rotates the mutable table and waits (bounded) until nothing immutable is left.
  bool flush_all(std::string* err) {
    {
      std::lock_guard<std::mutex> w(write_mu);
      if (!rotate(err)) return false;
    }
    if (!opt.background) {
      std::string e;
      while (flush_one(&e)) {}
      if (!e.empty()) { *err = e; return false; }
      return true;
    }
    std::unique_lock<std::mutex> l(mu);
    work_cv.notify_all();
    bool ok = done_cv.wait_for(l, std::chrono::seconds(120), [&] { return current->imm.empty() || !bg_error.empty(); });
    if (!bg_error.empty()) { *err = bg_error; return false; }
    if (!ok) { *err = "flush did not finish within 120 s"; return false; }
    return true;
  }

  // A sorted batch straight into a level-0 file, without the log (bulk loading).  What the memory tables hold is
  // flushed first, so the new file is the newest data.
  int ingest(const uint8_t* payload, size_t n, std::string* err) {
    if (opt.read_only) { *err = "the store is open read-only"; return -1; }
    std::vector<Op> ops;
    if (!parse_ops(payload, n, &ops)) { *err = "malformed batch"; return -1; }
    for (auto& op : ops) if (op.key.empty() || op.key.size() > 1024) { *err = "keys are 1 to 1024 bytes"; return -1; }
    if (ops.empty()) return 0;
    std::stable_sort(ops.begin(), ops.end(), [](const Op& a, const Op& b) { return a.key < b.key; });
    if (!flush_all(err)) return -1;
    std::lock_guard<std::mutex> w(write_mu);
    { std::lock_guard<std::mutex> l(mu); if (current->mem->bytes.load() || !current->imm.empty()) { *err = "a commit raced the bulk load; retry"; return -1; } }
    uint64_t num;
    { std::lock_guard<std::mutex> l(mu); num = next_file++; }
    TableBuilder b(table_path(num), opt.block_bytes);
    for (size_t i = 0; i < ops.size(); ++i) {
      if (i + 1 < ops.size() && ops[i + 1].key == ops[i].key) continue;  // the last write of a key wins
      b.add(ops[i].key, ops[i].kind, ops[i].value);
    }
    if (!b.finish(true)) { *err = "cannot write " + b.path; return -1; }
    auto t = std::make_shared<Table>();
    std::string e = t->open(b.path);
    if (!e.empty()) { *err = e; return -1; }
    t->number = num; t->level = 0;
    last_seq.fetch_add(ops.size());
    if (!publish({}, {t}, nullptr, err)) return -1;
    { std::lock_guard<std::mutex> l(mu); ++st.ingests; }
    work_cv.notify_all();
    return 0;
  }

  void close() {
    { std::lock_guard<std::mutex> l(mu); stopping = true; }
    work_cv.notify_all();
    if (flush_thread.joinable()) flush_thread.join();
    if (compact_thread.joinable()) compact_thread.join();
    if (wal_fd >= 0) { if (opt.sync) ::fdatasync(wal_fd); ::close(wal_fd); wal_fd = -1; }
    if (lock_fd >= 0) { ::flock(lock_fd, LOCK_UN); ::close(lock_fd); lock_fd = -1; }
  }
};

struct Snapshot {
  Store* store;
  std::shared_ptr<const Version> version;
  uint64_t seq;
  Bytes scratch;
};

struct Cursor {
  Snapshot* snap;
  Merged m;
  uint8_t ns;
  bool in_range() const { return m.valid && !m.key.empty() && uint8_t(m.key[0]) == ns; }
};

thread_local std::string g_error;

}  // namespace

extern "C" {

const char* afb_lsm_last_error() { return g_error.c_str(); }

// opts: memtable bytes, block bytes, target file bytes, level-1 bytes, level-0 files that start a merge, level-0
// files that delay commits, sync (0/1), read only (0/1), background threads (0/1); a zero keeps the default of
// the first six.
void* afb_lsm_open(const char* dir, const uint64_t* opts) {
  Options o;
  if (opts) {
    if (opts[0]) o.memtable_bytes = opts[0];
    if (opts[1]) o.block_bytes = opts[1];
    if (opts[2]) o.target_file_bytes = opts[2];
    if (opts[3]) o.level1_bytes = opts[3];
    if (opts[4]) o.l0_compact = int(opts[4]);
    if (opts[5]) o.l0_stall = int(opts[5]);
    o.sync = int(opts[6]); o.read_only = int(opts[7]); o.background = int(opts[8]);
  }
  auto* s = new Store();
  std::string e = s->open(dir, o);
  if (!e.empty()) { g_error = e; s->close(); delete s; return nullptr; }
  return s;
}

void afb_lsm_close(void* h) {
  auto* s = static_cast<Store*>(h);
  s->close();
  delete s;
}

int afb_lsm_write(void* h, const uint8_t* payload, uint64_t n) { return static_cast<Store*>(h)->write(payload, n, &g_error); }
int afb_lsm_ingest(void* h, const uint8_t* payload, uint64_t n) { return static_cast<Store*>(h)->ingest(payload, n, &g_error); }
int afb_lsm_flush(void* h) { return static_cast<Store*>(h)->flush_all(&g_error) ? 0 : -1; }

// full != 0: everything is merged into one level (deletes and shadowed rows disappear); else: until no level is
// over its budget.
int afb_lsm_compact(void* h, int full) {
  auto* s = static_cast<Store*>(h);
  if (!s->flush_all(&g_error)) return -1;
  std::string e;
  if (full) { s->compact_one(true, &e); }
  else while (s->compact_one(false, &e)) {}
  if (!e.empty()) { g_error = e; return -1; }
  return 0;
}

void afb_lsm_stats(void* h, uint64_t* out, int n) {
  auto* s = static_cast<Store*>(h);
  Stats st;
  std::shared_ptr<const Version> v;
  { std::lock_guard<std::mutex> l(s->mu); st = s->st; v = s->current; }
  st.mutable_bytes = v->mem->bytes.load();
  st.immutable_bytes = 0;
  for (auto& m : v->imm) st.immutable_bytes += m->bytes.load();
  st.immutable_tables = v->imm.size();
  st.bloom_skips = 0;
  for (int l = 0; l < kLevels; ++l) {
    st.level_files[l] = v->levels[l].size();
    st.level_bytes[l] = 0;
    for (auto& t : v->levels[l]) { st.level_bytes[l] += t->bytes; st.bloom_skips += t->bloom_skips.load(); }
  }
  st.last_sequence = s->last_seq.load();
  { std::lock_guard<std::mutex> l(s->snap_mu); st.live_snapshots = s->snapshots.size(); }
  const uint64_t* f = reinterpret_cast<const uint64_t*>(&st);
  for (int i = 0; i < n && i < int(sizeof(Stats) / 8); ++i) out[i] = f[i];
}

void* afb_lsm_snapshot(void* h) {
  auto* s = static_cast<Store*>(h);
  auto* sn = new Snapshot();
  sn->store = s;
  std::lock_guard<std::mutex> g(s->snap_mu);
  { std::lock_guard<std::mutex> l(s->mu); sn->version = s->current; }
  sn->seq = s->last_seq.load();
  s->snapshots.insert(sn->seq);
  return sn;
}

void afb_lsm_snapshot_free(void* h) {
  auto* sn = static_cast<Snapshot*>(h);
  {
    std::lock_guard<std::mutex> g(sn->store->snap_mu);
    auto it = sn->store->snapshots.find(sn->seq);
    if (it != sn->store->snapshots.end()) sn->store->snapshots.erase(it);
  }
  delete sn;
}

// 1: found (*val / *vlen valid until the snapshot's next call), 0: absent, -1: error
int afb_lsm_get(void* h, int ns, const uint8_t* key, uint64_t klen, const uint8_t** val, uint64_t* vlen) {
  auto* sn = static_cast<Snapshot*>(h);
  Bytes k(1, char(ns));
  k.append(reinterpret_cast<const char*>(key), klen);
  std::string e;
  int r = sn->version->get(k, sn->seq, &sn->scratch, &e);
  if (r < 0) { g_error = e; return -1; }
  if (r == 1) { *val = reinterpret_cast<const uint8_t*>(sn->scratch.data()); *vlen = sn->scratch.size(); }
  return r;
}

void* afb_lsm_cursor(void* h, int ns) {
  auto* sn = static_cast<Snapshot*>(h);
  auto* c = new Cursor();
  c->snap = sn;
  c->ns = uint8_t(ns);
  sn->version->sources(sn->seq, &c->m.src);
  return c;
}

void afb_lsm_cursor_free(void* h) { delete static_cast<Cursor*>(h); }

// op: 0 first, 1 last, 2 next, 3 previous, 4 first key >= key, 5 last key <= key.  1: on an entry, 0: off the
// end of the namespace, -1: a damaged file.
int afb_lsm_cursor_move(void* h, int op, const uint8_t* key, uint64_t klen) {
  auto* c = static_cast<Cursor*>(h);
  Bytes k(1, char(c->ns));
  if (key) k.append(reinterpret_cast<const char*>(key), klen);
  switch (op) {
    case 0: c->m.seek_ge(Bytes(1, char(c->ns))); break;
    case 1: {
      if (c->ns == 255) { c->m.seek_le(Bytes(2048, char(0xFF))); break; }
      Bytes upper(1, char(c->ns + 1));
      c->m.seek_le(upper);
      if (c->m.valid && c->m.key == upper) c->m.prev();
      break;
    }
    case 2: if (!c->in_range()) return 0; c->m.next(); break;
    case 3: if (!c->in_range()) return 0; c->m.prev(); break;
    case 4: c->m.seek_ge(k); break;
    case 5: c->m.seek_le(k); break;
    default: g_error = "unknown cursor operation"; return -1;
  }
  if (!c->m.error.empty()) { g_error = c->m.error; return -1; }
  return c->in_range() ? 1 : 0;
}

void afb_lsm_cursor_entry(void* h, const uint8_t** key, uint64_t* klen, const uint8_t** val, uint64_t* vlen) {
  auto* c = static_cast<Cursor*>(h);
  *key = reinterpret_cast<const uint8_t*>(c->m.key.data()) + 1;
  *klen = c->m.key.size() - 1;
  *val = c->m.val;
  *vlen = c->m.vlen;
}

}  // extern "C"
