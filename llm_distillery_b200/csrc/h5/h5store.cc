// Minimal HDF5 container for teacher-distribution datasets, written from the file-format specification
// (no libhdf5 on the target image). Produces "earliest"-format files that stock HDF5 / h5py read:
//   superblock v0, old-style groups (v1 B-tree + local heap + symbol-table nodes), v1 object headers,
//   chunked datasets (v1 chunk B-tree, one chunk per dataset) with the deflate filter, scalar attributes with
//   variable-length UTF-8 strings in global-heap collections and 64-bit integers.
// Layout:  /                 attrs vocab_family (str), topk (int64)
//          /convo_<id>/      attrs content_sha (str), sample (str)
//              distributions float16 [rows, cols]  gzip
//              indices       uint32  [rows, cols]  gzip   (absent for full-vocabulary distributions)
//
// Mutation model: data objects are append-only; the root group's link structures (heap, symbol nodes, B-tree)
// and the root object header are rewritten at the end of the file on flush, and the superblock is rewritten
// last (after fsync), so a kill at any moment leaves the previous consistent state readable. Deleted or replaced
// objects become dead space until repack(). The reader walks real B-trees / heaps / continuation blocks and
// also understands contiguous and multi-chunk datasets and fixed-length string attributes, so files produced by
// stock HDF5 with the same logical layout load as well.
#include <zlib.h>

#include <algorithm>
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <deque>
#include <functional>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

namespace {

constexpr uint64_t UNDEF = ~0ull;
constexpr int GROUP_LEAF_K = 16;      // symbol-table node holds up to 2K = 32 entries
constexpr int GROUP_INTERNAL_K = 16;  // group B-tree node holds up to 2K = 32 children
constexpr int CHUNK_K = 32;           // fixed for superblock v0
constexpr int SUB_LEAF_K = 4, SUB_INTERNAL_K = 16;  // only matter for node sizes of per-conversation groups

struct Buf {
  std::vector<uint8_t> b;
  void u8(uint8_t v) { b.push_back(v); }
  void u16(uint16_t v) { for (int i = 0; i < 2; ++i) b.push_back((v >> (8 * i)) & 0xff); }
  void u32(uint32_t v) { for (int i = 0; i < 4; ++i) b.push_back((v >> (8 * i)) & 0xff); }
  void u64(uint64_t v) { for (int i = 0; i < 8; ++i) b.push_back((v >> (8 * i)) & 0xff); }
  void bytes(const void* p, size_t n) { const uint8_t* q = (const uint8_t*)p; b.insert(b.end(), q, q + n); }
  void zeros(size_t n) { b.insert(b.end(), n, 0); }
  void pad8() { while (b.size() & 7) b.push_back(0); }
  size_t size() const { return b.size(); }
};

uint16_t rd16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }
uint32_t rd32(const uint8_t* p) { return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24); }
uint64_t rd64(const uint8_t* p) { return (uint64_t)rd32(p) | ((uint64_t)rd32(p + 4) << 32); }

// ---------------------------------------------------------------- datatype / dataspace message bodies
void dt_f16(Buf& o) {  // IEEE half, little endian
  o.u8(0x11); o.u8(0x20); o.u8(15); o.u8(0); o.u32(2);
  o.u16(0); o.u16(16); o.u8(10); o.u8(5); o.u8(0); o.u8(10); o.u32(15);
}
void dt_uint(Buf& o, int size, bool is_signed) {
  o.u8(0x10); o.u8(is_signed ? 0x08 : 0x00); o.u8(0); o.u8(0); o.u32(size);
  o.u16(0); o.u16((uint16_t)(size * 8));
}
void dt_vlen_utf8(Buf& o) {
  o.u8(0x19); o.u8(0x01); o.u8(0x01); o.u8(0); o.u32(16);  // class 9 v1; type=string, pad=nullterm; cset=UTF-8
  dt_uint(o, 1, false);                                    // base type: 1-byte unsigned
}
void ds_simple(Buf& o, const std::vector<uint64_t>& dims) {
  o.u8(1); o.u8((uint8_t)dims.size()); o.u8(0); o.u8(0); o.u32(0);
  for (auto d : dims) o.u64(d);
}

struct Msg { uint16_t type; std::vector<uint8_t> data; };

void add_msg(std::vector<Msg>& ms, uint16_t type, Buf& body) {
  body.pad8();
  ms.push_back({type, body.b});
}

std::vector<uint8_t> object_header_v1(const std::vector<Msg>& ms) {
  Buf body;
  for (auto& m : ms) {
    body.u16(m.type); body.u16((uint16_t)m.data.size()); body.u8(0); body.u8(0); body.u8(0); body.u8(0);
    body.bytes(m.data.data(), m.data.size());
  }
  Buf h;
  h.u8(1); h.u8(0); h.u16((uint16_t)ms.size()); h.u32(1); h.u32((uint32_t)body.size()); h.u32(0);  // 16-byte prefix
  h.bytes(body.b.data(), body.size());
  return h.b;
}

Msg attr_msg(const std::string& name, std::function<void(Buf&)> dtype, const std::vector<uint8_t>& data) {
  Buf dt; dtype(dt);
  Buf ds; ds_simple(ds, {});
  Buf a;
  a.u8(1); a.u8(0); a.u16((uint16_t)(name.size() + 1)); a.u16((uint16_t)dt.size()); a.u16((uint16_t)ds.size());
  a.bytes(name.c_str(), name.size() + 1); a.pad8();
  a.bytes(dt.b.data(), dt.size()); a.pad8();
  a.bytes(ds.b.data(), ds.size()); a.pad8();
  a.bytes(data.data(), data.size());
  a.pad8();
  return {0x000C, a.b};
}

// ---------------------------------------------------------------- the store
struct DatasetInfo { uint64_t rows = 0, cols = 0; int elem = 0; bool found = false; };

struct Store {
  int fd = -1;
  std::string path;
  uint64_t eof = 0;
  std::map<std::string, uint64_t> links;   // root link name -> object header address
  std::map<std::string, std::string> root_str_attrs;
  std::map<std::string, int64_t> root_int_attrs;
  bool dirty = false;
  std::string err;
  std::mutex mu;  // protects links / eof / fd writes

  // -------- raw IO
  bool pread_all(uint64_t off, void* dst, size_t n) {
    uint8_t* p = (uint8_t*)dst;
    while (n) {
      ssize_t r = ::pread(fd, p, n, (off_t)off);
      if (r <= 0) { err = "short read at " + std::to_string(off); return false; }
      p += r; off += r; n -= r;
    }
    return true;
  }
  bool pwrite_all(uint64_t off, const void* src, size_t n) {
    const uint8_t* p = (const uint8_t*)src;
    while (n) {
      ssize_t r = ::pwrite(fd, p, n, (off_t)off);
      if (r <= 0) { err = "write failed at " + std::to_string(off); return false; }
      p += r; off += r; n -= r;
    }
    return true;
  }
  uint64_t append(const void* src, size_t n) {  // 8-byte aligned append; returns address
    eof = (eof + 7) & ~7ull;
    uint64_t at = eof;
    if (!pwrite_all(at, src, n)) return UNDEF;
    eof += n;
    return at;
  }

  // -------- global heap collection holding the given strings; returns address, ids are 1..n
  uint64_t write_gcol(const std::vector<std::string>& strs) {
    size_t need = 16;
    for (auto& s : strs) need += 16 + ((s.size() + 7) & ~7ull);
    size_t size = std::max<size_t>(4096, (need + 16 + 7) & ~7ull);
    Buf g;
    g.bytes("GCOL", 4); g.u8(1); g.u8(0); g.u8(0); g.u8(0); g.u64(size);
    uint16_t idx = 1;
    for (auto& s : strs) {
      g.u16(idx++); g.u16(1); g.u32(0); g.u64(s.size());
      g.bytes(s.data(), s.size()); g.pad8();
    }
    size_t rem = size - g.size();
    if (rem >= 16) { g.u16(0); g.u16(0); g.u32(0); g.u64(rem); g.zeros(rem - 16); }
    else g.zeros(rem);
    return append(g.b.data(), g.size());
  }
  static std::vector<uint8_t> vlen_ref(uint32_t len, uint64_t gcol, uint32_t idx) {
    Buf r; r.u32(len); r.u64(gcol); r.u32(idx); return r.b;
  }

  // -------- one chunked+deflated dataset (single chunk). `comp` is the already-deflated payload.
  // `shuffled`: the payload was byte-shuffled (HDF5 filter 2) before deflate; the filter pipeline message says so.
  uint64_t write_dataset(uint64_t rows, uint64_t cols, int elem, bool is_f16, const std::vector<uint8_t>& comp,
                         bool shuffled = false, int level = 6) {
    uint64_t chunk_addr = append(comp.data(), comp.size());
    if (chunk_addr == UNDEF) return UNDEF;
    // chunk B-tree: one leaf node with one entry
    const int rank1 = 3;
    const size_t keysz = 8 + 8 * rank1;
    Buf t;
    t.bytes("TREE", 4); t.u8(1); t.u8(0); t.u16(1); t.u64(UNDEF); t.u64(UNDEF);
    t.u32((uint32_t)comp.size()); t.u32(0); t.u64(0); t.u64(0); t.u64(0);   // key 0
    t.u64(chunk_addr);                                                     // child 0
    t.u32(0); t.u32(0); t.u64(rows); t.u64(0); t.u64(0);                    // key 1 (past the end)
    size_t full = 24 + (2 * CHUNK_K + 1) * keysz + 2 * CHUNK_K * 8;
    t.zeros(full - t.size());
    uint64_t tree_addr = append(t.b.data(), t.size());
    if (tree_addr == UNDEF) return UNDEF;
    std::vector<Msg> ms;
    { Buf m; ds_simple(m, {rows, cols}); add_msg(ms, 0x0001, m); }
    { Buf m; if (is_f16) dt_f16(m); else dt_uint(m, elem, false); add_msg(ms, 0x0003, m); }
    { Buf m; m.u8(2); m.u8(3); m.u8(2); m.u8(0); add_msg(ms, 0x0005, m); }
    { Buf m; m.u8(1); m.u8(shuffled ? 2 : 1); m.zeros(6);
      if (shuffled) { m.u16(2); m.u16(0); m.u16(1); m.u16(1); m.u32((uint32_t)elem); m.u32(0); }   // shuffle(elem size)
      m.u16(1); m.u16(0); m.u16(1); m.u16(1); m.u32((uint32_t)level); m.u32(0);                      // deflate(level)
      add_msg(ms, 0x000B, m); }
    { Buf m; m.u8(3); m.u8(2); m.u8(rank1); m.u64(tree_addr); m.u32((uint32_t)rows); m.u32((uint32_t)cols);
      m.u32((uint32_t)elem); add_msg(ms, 0x0008, m); }
    auto h = object_header_v1(ms);
    return append(h.data(), h.size());
  }

  // -------- old-style group: local heap + symbol nodes + B-tree + object header. Returns header address and,
  // through btree/heap, the addresses cached in the parent's symbol-table entry.
  struct GroupAddrs { uint64_t header, btree, heap; };
  GroupAddrs write_group(const std::vector<std::pair<std::string, uint64_t>>& sorted_links,
                         const std::map<std::string, std::pair<uint64_t, uint64_t>>* child_cache,
                         const std::vector<Msg>& extra_msgs, int leaf_k, int internal_k) {
    GroupAddrs ga{UNDEF, UNDEF, UNDEF};
    // local heap: offset 0 is the empty string
    Buf data; data.zeros(8);
    std::vector<uint64_t> name_off;
    for (auto& kv : sorted_links) {
      name_off.push_back(data.size());
      data.bytes(kv.first.c_str(), kv.first.size() + 1); data.pad8();
    }
    Buf hp;
    hp.bytes("HEAP", 4); hp.u8(0); hp.u8(0); hp.u8(0); hp.u8(0);
    hp.u64(data.size()); hp.u64(1);  // free-list head: 1 = no free block
    eof = (eof + 7) & ~7ull;
    uint64_t heap_addr = eof;
    hp.u64(heap_addr + 32);
    hp.bytes(data.b.data(), data.size());
    if (append(hp.b.data(), hp.size()) == UNDEF) return ga;
    // symbol-table nodes
    const size_t per = 2 * (size_t)leaf_k;
    struct Child { uint64_t addr; uint64_t maxkey; };
    std::vector<Child> level;
    size_t n = sorted_links.size();
    for (size_t i = 0; i < n; i += per) {
      size_t cnt = std::min(per, n - i);
      Buf s;
      s.bytes("SNOD", 4); s.u8(1); s.u8(0); s.u16((uint16_t)cnt);
      for (size_t j = 0; j < cnt; ++j) {
        auto& kv = sorted_links[i + j];
        s.u64(name_off[i + j]); s.u64(kv.second);
        const std::pair<uint64_t, uint64_t>* cc = nullptr;
        if (child_cache) { auto it = child_cache->find(kv.first); if (it != child_cache->end()) cc = &it->second; }
        if (cc) { s.u32(1); s.u32(0); s.u64(cc->first); s.u64(cc->second); }
        else { s.u32(0); s.u32(0); s.u64(0); s.u64(0); }
      }
      s.zeros(8 + per * 40 - s.size());
      uint64_t a = append(s.b.data(), s.size());
      if (a == UNDEF) return ga;
      level.push_back({a, name_off[i + cnt - 1]});
    }
    // B-tree levels, bottom-up
    const size_t fan = 2 * (size_t)internal_k;
    const size_t node_full = 24 + (fan + 1) * 8 + fan * 8;
    int lvl = 0;
    if (level.empty()) {  // empty group: a leaf node with no entries
      Buf t;
      t.bytes("TREE", 4); t.u8(0); t.u8(0); t.u16(0); t.u64(UNDEF); t.u64(UNDEF);
      t.zeros(node_full - t.size());
      ga.btree = append(t.b.data(), t.size());
      if (ga.btree == UNDEF) return ga;
    }
    while (!level.empty()) {
      std::vector<Child> up;
      std::vector<uint64_t> addrs;
      // pre-compute node addresses of this level so siblings can be linked
      size_t nodes = (level.size() + fan - 1) / fan;
      eof = (eof + 7) & ~7ull;
      for (size_t k = 0; k < nodes; ++k) addrs.push_back(eof + k * ((node_full + 7) & ~7ull));
      for (size_t k = 0; k < nodes; ++k) {
        size_t lo = k * fan, cnt = std::min(fan, level.size() - lo);
        Buf t;
        t.bytes("TREE", 4); t.u8(0); t.u8((uint8_t)lvl); t.u16((uint16_t)cnt);
        t.u64(k ? addrs[k - 1] : UNDEF); t.u64(k + 1 < nodes ? addrs[k + 1] : UNDEF);
        t.u64(lo ? level[lo - 1].maxkey : 0);  // key 0: everything in child 0 is greater than this name
        for (size_t j = 0; j < cnt; ++j) { t.u64(level[lo + j].addr); t.u64(level[lo + j].maxkey); }
        t.zeros(node_full - t.size());
        if (append(t.b.data(), t.size()) == UNDEF) return ga;
        up.push_back({addrs[k], level[lo + cnt - 1].maxkey});
      }
      if (up.size() == 1) { ga.btree = up[0].addr; break; }
      level.swap(up);
      ++lvl;
    }
    ga.heap = heap_addr;
    std::vector<Msg> ms;
    { Buf m; m.u64(ga.btree); m.u64(ga.heap); add_msg(ms, 0x0011, m); }
    for (auto& e : extra_msgs) ms.push_back(e);
    auto h = object_header_v1(ms);
    ga.header = append(h.data(), h.size());
    return ga;
  }

  // -------- conversation group
  std::map<std::string, std::pair<uint64_t, uint64_t>> group_cache;  // root link -> (btree, heap) for new groups

  bool put_group(const std::string& name, uint64_t distr_hdr, uint64_t idx_hdr, const std::string& sha,
                 const std::string& sample) {
    uint64_t gcol = write_gcol({sha, sample});
    if (gcol == UNDEF) return false;
    std::vector<Msg> attrs;
    attrs.push_back(attr_msg("content_sha", dt_vlen_utf8, vlen_ref((uint32_t)sha.size(), gcol, 1)));
    attrs.push_back(attr_msg("sample", dt_vlen_utf8, vlen_ref((uint32_t)sample.size(), gcol, 2)));
    std::vector<std::pair<std::string, uint64_t>> ls;
    ls.push_back({"distributions", distr_hdr});
    if (idx_hdr != UNDEF) ls.push_back({"indices", idx_hdr});
    std::sort(ls.begin(), ls.end());
    GroupAddrs ga = write_group(ls, nullptr, attrs, SUB_LEAF_K, SUB_INTERNAL_K);
    if (ga.header == UNDEF) return false;
    links[name] = ga.header;
    group_cache[name] = {ga.btree, ga.heap};
    dirty = true;
    return true;
  }

  // -------- flush: new root structures, then superblock
  bool flush() {
    if (!dirty && eof >= 96) return true;
    std::vector<std::pair<std::string, uint64_t>> ls(links.begin(), links.end());  // std::map iterates in byte order
    std::vector<std::string> strs;
    std::vector<Msg> attrs;
    for (auto& kv : root_str_attrs) strs.push_back(kv.second);
    uint64_t gcol = UNDEF;
    if (!strs.empty()) { gcol = write_gcol(strs); if (gcol == UNDEF) return false; }
    uint32_t i = 1;
    for (auto& kv : root_str_attrs) attrs.push_back(attr_msg(kv.first, dt_vlen_utf8, vlen_ref((uint32_t)kv.second.size(), gcol, i++)));
    for (auto& kv : root_int_attrs) {
      Buf d; d.u64((uint64_t)kv.second);
      attrs.push_back(attr_msg(kv.first, [](Buf& o) { dt_uint(o, 8, true); }, d.b));
    }
    // only cache (btree, heap) for links whose group we still know; others get cache type 0
    std::map<std::string, std::pair<uint64_t, uint64_t>> cache;
    for (auto& kv : group_cache) { auto it = links.find(kv.first); if (it != links.end()) cache[kv.first] = kv.second; }
    GroupAddrs ga = write_group(ls, &cache, attrs, GROUP_LEAF_K, GROUP_INTERNAL_K);
    if (ga.header == UNDEF) return false;
    eof = (eof + 7) & ~7ull;
    if (::ftruncate(fd, (off_t)eof) != 0) { err = "ftruncate failed"; return false; }
    if (::fsync(fd) != 0) { err = "fsync failed"; return false; }
    Buf sb;
    const uint8_t sig[8] = {0x89, 'H', 'D', 'F', '\r', '\n', 0x1a, '\n'};
    sb.bytes(sig, 8);
    sb.u8(0); sb.u8(0); sb.u8(0); sb.u8(0); sb.u8(0); sb.u8(8); sb.u8(8); sb.u8(0);
    sb.u16(GROUP_LEAF_K); sb.u16(GROUP_INTERNAL_K); sb.u32(0);
    sb.u64(0); sb.u64(UNDEF); sb.u64(eof); sb.u64(UNDEF);
    sb.u64(0); sb.u64(ga.header); sb.u32(1); sb.u32(0); sb.u64(ga.btree); sb.u64(ga.heap);
    if (!pwrite_all(0, sb.b.data(), sb.size())) return false;
    if (::fsync(fd) != 0) { err = "fsync failed"; return false; }
    dirty = false;
    return true;
  }

  // ================================================================ reader
  struct ParsedMsg { uint16_t type; std::vector<uint8_t> data; };

  bool read_header(uint64_t addr, std::vector<ParsedMsg>& out) {
    uint8_t pre[16];
    if (!pread_all(addr, pre, 16)) return false;
    if (pre[0] != 1) { err = "unsupported object header version " + std::to_string(pre[0]); return false; }
    uint16_t nmsg = rd16(pre + 2);
    uint32_t size = rd32(pre + 8);
    std::deque<std::pair<uint64_t, uint64_t>> blocks;
    blocks.push_back({addr + 16, size});
    while (!blocks.empty() && out.size() < (size_t)nmsg + 64) {
      auto blk = blocks.front(); blocks.pop_front();
      std::vector<uint8_t> b(blk.second);
      if (blk.second && !pread_all(blk.first, b.data(), b.size())) return false;
      size_t p = 0;
      while (p + 8 <= b.size()) {
        uint16_t type = rd16(&b[p]); uint16_t sz = rd16(&b[p + 2]);
        p += 8;
        if (p + sz > b.size()) break;
        if (type == 0x0010 && sz >= 16) blocks.push_back({rd64(&b[p]), rd64(&b[p + 8])});
        else if (type != 0) out.push_back({type, std::vector<uint8_t>(b.begin() + p, b.begin() + p + sz)});
        p += sz;
      }
    }
    return true;
  }

  bool read_heap_name(uint64_t heap_data_addr, uint64_t off, std::string& name) {
    char buf[256];
    name.clear();
    uint64_t at = heap_data_addr + off;
    while (true) {
      ssize_t r = ::pread(fd, buf, sizeof(buf), (off_t)at);
      if (r <= 0) { err = "heap name read failed"; return false; }
      for (ssize_t i = 0; i < r; ++i) { if (!buf[i]) return true; name.push_back(buf[i]); }
      at += r;
      if (name.size() > 65536) { err = "unterminated heap name"; return false; }
    }
  }

  bool walk_group_btree(uint64_t node, uint64_t heap_data, std::map<std::string, uint64_t>& out, int depth = 0) {
    if (node == UNDEF || depth > 16) return true;
    uint8_t h[24];
    if (!pread_all(node, h, 24)) return false;
    if (!memcmp(h, "SNOD", 4)) {
      uint16_t n = rd16(h + 6);
      std::vector<uint8_t> e((size_t)n * 40);
      if (n && !pread_all(node + 8, e.data(), e.size())) return false;
      for (uint16_t i = 0; i < n; ++i) {
        std::string name;
        if (!read_heap_name(heap_data, rd64(&e[i * 40]), name)) return false;
        out[name] = rd64(&e[i * 40 + 8]);
      }
      return true;
    }
    if (memcmp(h, "TREE", 4)) { err = "bad group node signature"; return false; }
    uint16_t used = rd16(h + 6);
    std::vector<uint8_t> body((size_t)used * 16 + 8);
    if (!pread_all(node + 24, body.data(), body.size())) return false;
    for (uint16_t i = 0; i < used; ++i)
      if (!walk_group_btree(rd64(&body[8 + i * 16]), heap_data, out, depth + 1)) return false;
    return true;
  }

  bool read_group_links(const std::vector<ParsedMsg>& ms, std::map<std::string, uint64_t>& out) {
    for (auto& m : ms) {
      if (m.type == 0x0011 && m.data.size() >= 16) {
        uint64_t bt = rd64(&m.data[0]), hp = rd64(&m.data[8]);
        uint8_t hh[32];
        if (!pread_all(hp, hh, 32)) return false;
        if (memcmp(hh, "HEAP", 4)) { err = "bad local heap"; return false; }
        return walk_group_btree(bt, rd64(hh + 24), out);
      }
    }
    err = "group has no symbol table message (new-style groups are not supported)";
    return false;
  }

  bool read_gheap_obj(uint64_t gcol, uint32_t idx, std::string& out) {
    uint8_t h[16];
    if (!pread_all(gcol, h, 16)) return false;
    if (memcmp(h, "GCOL", 4)) { err = "bad global heap"; return false; }
    uint64_t size = rd64(h + 8);
    std::vector<uint8_t> b(size);
    if (!pread_all(gcol, b.data(), size)) return false;
    size_t p = 16;
    while (p + 16 <= size) {
      uint16_t id = rd16(&b[p]); uint64_t sz = rd64(&b[p + 8]);
      if (id == 0) break;
      if (id == idx) { if (p + 16 + sz > size) break; out.assign((const char*)&b[p + 16], sz); return true; }
      p += 16 + ((sz + 7) & ~7ull);
    }
    err = "global heap object not found";
    return false;
  }

  // attribute value as string (vlen or fixed) or integer
  bool parse_attr(const std::vector<uint8_t>& d, std::string& name, std::string& sval, int64_t& ival, bool& is_str) {
    if (d.size() < 8) return false;
    int ver = d[0];
    size_t p; uint16_t nsz, dtsz, dssz;
    nsz = rd16(&d[2]); dtsz = rd16(&d[4]); dssz = rd16(&d[6]);
    p = 8;
    if (ver == 3) p = 9;
    auto adv = [&](size_t n) { return ver == 1 ? ((n + 7) & ~7ull) : n; };
    if (p + nsz > d.size()) return false;
    name.assign((const char*)&d[p], strnlen((const char*)&d[p], nsz));
    p += adv(nsz);
    if (p + dtsz > d.size()) return false;
    const uint8_t* dt = &d[p];
    int cls = dt[0] & 0x0f;
    uint32_t tsize = rd32(dt + 4);
    p += adv(dtsz);
    p += adv(dssz);
    if (p > d.size()) return false;
    const uint8_t* val = &d[p];
    size_t left = d.size() - p;
    is_str = false;
    if (cls == 9 && (dt[1] & 0x0f) == 1) {
      if (left < 16) return false;
      is_str = true;
      uint32_t len = rd32(val);
      if (len == 0) { sval.clear(); return true; }
      if (!read_gheap_obj(rd64(val + 4), rd32(val + 12), sval)) return false;
      if (sval.size() > len) sval.resize(len);
      return true;
    }
    if (cls == 3) {
      is_str = true;
      sval.assign((const char*)val, strnlen((const char*)val, std::min<size_t>(tsize, left)));
      return true;
    }
    if (cls == 0 && tsize <= 8 && left >= tsize) {
      uint64_t v = 0;
      for (uint32_t i = 0; i < tsize; ++i) v |= (uint64_t)val[i] << (8 * i);
      if ((dt[1] & 0x08) && tsize < 8 && (v >> (8 * tsize - 1))) v |= ~0ull << (8 * tsize);
      ival = (int64_t)v;
      return true;
    }
    return false;
  }

  bool read_attrs(uint64_t hdr, std::map<std::string, std::string>& strs, std::map<std::string, int64_t>& ints) {
    std::vector<ParsedMsg> ms;
    if (!read_header(hdr, ms)) return false;
    for (auto& m : ms) {
      if (m.type != 0x000C) continue;
      std::string n, s; int64_t iv = 0; bool is_str = false;
      if (parse_attr(m.data, n, s, iv, is_str)) { if (is_str) strs[n] = s; else ints[n] = iv; }
    }
    return true;
  }

  // chunk B-tree walk
  struct ChunkRef { uint64_t addr; uint32_t size; uint32_t mask; std::vector<uint64_t> off; };
  bool walk_chunks(uint64_t node, int rank1, std::vector<ChunkRef>& out, int depth = 0) {
    if (node == UNDEF || depth > 16) return true;
    uint8_t h[24];
    if (!pread_all(node, h, 24)) return false;
    if (memcmp(h, "TREE", 4) || h[4] != 1) { err = "bad chunk B-tree node"; return false; }
    int level = h[5];
    uint16_t used = rd16(h + 6);
    size_t keysz = 8 + 8 * (size_t)rank1;
    std::vector<uint8_t> body((size_t)used * (keysz + 8) + keysz);
    if (!pread_all(node + 24, body.data(), body.size())) return false;
    for (uint16_t i = 0; i < used; ++i) {
      const uint8_t* k = &body[i * (keysz + 8)];
      uint64_t child = rd64(k + keysz);
      if (level > 0) { if (!walk_chunks(child, rank1, out, depth + 1)) return false; continue; }
      ChunkRef c{child, rd32(k), rd32(k + 4), {}};
      for (int d = 0; d < rank1; ++d) c.off.push_back(rd64(k + 8 + 8 * d));
      out.push_back(c);
    }
    return true;
  }

  bool read_dataset(uint64_t hdr, std::vector<uint8_t>& raw, DatasetInfo& info) {
    std::vector<ParsedMsg> ms;
    if (!read_header(hdr, ms)) return false;
    std::vector<uint64_t> dims;
    int elem = 0, layout_class = -1, rank1 = 0;
    uint64_t data_addr = UNDEF, data_size = 0;
    std::vector<uint32_t> cdims;
    bool deflate = false, shuffle = false;
    std::vector<uint8_t> compact;
    for (auto& m : ms) {
      const auto& d = m.data;
      if (m.type == 0x0001 && d.size() >= 8) {
        int ver = d[0], rank = d[1];
        size_t p = ver == 1 ? 8 : 4;
        for (int i = 0; i < rank && p + 8 <= d.size(); ++i, p += 8) dims.push_back(rd64(&d[p]));
      } else if (m.type == 0x0003 && d.size() >= 8) {
        elem = (int)rd32(&d[4]);
      } else if (m.type == 0x0008 && d.size() >= 2) {
        if (d[0] != 3) { err = "unsupported data layout version"; return false; }
        layout_class = d[1];
        if (layout_class == 2) {
          rank1 = d[2]; data_addr = rd64(&d[3]);
          for (int i = 0; i < rank1; ++i) cdims.push_back(rd32(&d[11 + 4 * i]));
        } else if (layout_class == 1) { data_addr = rd64(&d[2]); data_size = rd64(&d[10]); }
        else if (layout_class == 0) { uint16_t sz = rd16(&d[2]); compact.assign(d.begin() + 4, d.begin() + 4 + sz); }
      } else if (m.type == 0x000B && d.size() >= 8) {
        int ver = d[0], nf = d[1];
        size_t p = ver == 1 ? 8 : 2;
        for (int f = 0; f < nf && p + 8 <= d.size(); ++f) {
          uint16_t id = rd16(&d[p]);
          uint16_t nlen = (ver == 1 || id >= 256) ? rd16(&d[p + 2]) : 0;
          size_t q = p + ((ver == 1 || id >= 256) ? 4 : 2);
          uint16_t ncd = rd16(&d[q + 2]);
          q += 4;
          q += ver == 1 ? ((nlen + 7) & ~7u) : nlen;
          q += 4 * (size_t)ncd;
          if (ver == 1 && (ncd & 1)) q += 4;
          if (id == 1) deflate = true; else if (id == 2) shuffle = true;
          else { err = "unsupported filter " + std::to_string(id); return false; }
          p = q;
        }
      }
    }
    if (dims.empty() || elem <= 0) { err = "dataset without dataspace/datatype"; return false; }
    while (dims.size() < 2) dims.push_back(1);
    info.rows = dims[0]; info.cols = 1;
    for (size_t i = 1; i < dims.size(); ++i) info.cols *= dims[i];
    info.elem = elem; info.found = true;
    const uint64_t total = info.rows * info.cols * (uint64_t)elem;
    raw.assign(total, 0);
    if (layout_class == 0) { memcpy(raw.data(), compact.data(), std::min<size_t>(total, compact.size())); return true; }
    if (layout_class == 1) { (void)data_size; return data_addr == UNDEF || total == 0 || pread_all(data_addr, raw.data(), total); }
    if (layout_class != 2 || dims.size() != 2 || rank1 != 3) { err = "unsupported dataset layout"; return false; }
    std::vector<ChunkRef> chunks;
    if (!walk_chunks(data_addr, rank1, chunks)) return false;
    const uint64_t crow = cdims[0], ccol = cdims[1];
    std::vector<uint8_t> cbuf, ubuf(crow * ccol * (uint64_t)elem), tmp;
    for (auto& c : chunks) {
      cbuf.resize(c.size);
      if (!pread_all(c.addr, cbuf.data(), c.size)) return false;
      const uint8_t* src = cbuf.data();
      if (deflate && !(c.mask & (shuffle ? 2u : 1u))) {
        uLongf dl = (uLongf)ubuf.size();
        if (uncompress(ubuf.data(), &dl, cbuf.data(), (uLong)c.size) != Z_OK) { err = "inflate failed"; return false; }
        src = ubuf.data();
      } else if (c.size < ubuf.size()) { err = "short uncompressed chunk"; return false; }
      if (shuffle && !(c.mask & 1u)) {
        tmp.resize(ubuf.size());
        size_t n = ubuf.size() / elem;
        for (size_t i = 0; i < n; ++i) for (int b = 0; b < elem; ++b) tmp[i * elem + b] = src[(size_t)b * n + i];
        src = tmp.data();
      }
      for (uint64_t r = 0; r < crow; ++r) {
        uint64_t gr = c.off[0] + r;
        if (gr >= info.rows) break;
        uint64_t gc = c.off[1];
        if (gc >= info.cols) break;
        uint64_t n = std::min<uint64_t>(ccol, info.cols - gc);
        memcpy(&raw[(gr * info.cols + gc) * elem], src + r * ccol * elem, n * elem);
      }
    }
    return true;
  }

  // -------- open / create
  bool open(const char* p, bool create) {
    path = p;
    fd = ::open(p, create ? (O_RDWR | O_CREAT) : O_RDWR, 0644);
    if (fd < 0) { fd = ::open(p, O_RDONLY); if (fd < 0) { err = std::string("cannot open ") + p; return false; } }
    struct stat st;
    fstat(fd, &st);
    if (st.st_size == 0) { eof = 96; dirty = true; return flush(); }
    uint8_t sb[96];
    if (st.st_size < 96 || !pread_all(0, sb, 96)) { err = "file too small for an HDF5 superblock"; return false; }
    const uint8_t sig[8] = {0x89, 'H', 'D', 'F', '\r', '\n', 0x1a, '\n'};
    if (memcmp(sb, sig, 8)) { err = "not an HDF5 file"; return false; }
    if (sb[8] > 1 || sb[13] != 8 || sb[14] != 8) { err = "unsupported superblock (need v0/v1 with 8-byte offsets)"; return false; }
    size_t o = sb[8] == 1 ? 28 : 24;  // v1 has 4 more bytes (indexed storage K + reserved)
    if (sb[8] == 1 && !pread_all(0, sb, 96)) return false;
    uint8_t sb2[100];
    if (!pread_all(0, sb2, std::min<size_t>(100, st.st_size))) return false;
    uint64_t file_eof = rd64(sb2 + o + 16);
    uint64_t root_hdr = rd64(sb2 + o + 32 + 8);
    eof = std::min<uint64_t>(file_eof, (uint64_t)st.st_size);
    std::vector<ParsedMsg> ms;
    if (!read_header(root_hdr, ms)) return false;
    if (!read_group_links(ms, links)) return false;
    if (!read_attrs(root_hdr, root_str_attrs, root_int_attrs)) return false;
    dirty = false;
    return true;
  }
};

// Byte shuffle (HDF5 filter 2): all first bytes of the elements, then all second bytes, ... Slowly varying high
// bytes (sorted fp16 log-probs, token ids below 2^17) then form long runs, which deflate packs better and faster.
void shuffle_bytes(const uint8_t* src, size_t n_elem, int elem, std::vector<uint8_t>& out) {
  out.resize(n_elem * (size_t)elem);
  for (int b = 0; b < elem; ++b) {
    uint8_t* d = out.data() + (size_t)b * n_elem;
    const uint8_t* sp = src + b;
    for (size_t i = 0; i < n_elem; ++i) d[i] = sp[i * (size_t)elem];
  }
}

bool deflate_buf(const void* src, size_t n, int level, std::vector<uint8_t>& out) {
  uLongf cap = compressBound((uLong)n);
  out.resize(cap);
  if (compress2(out.data(), &cap, (const Bytef*)src, (uLong)n, level) != Z_OK) return false;
  out.resize(cap);
  return true;
}

std::string convo_name(long long id) { return "convo_" + std::to_string(id); }

void copy_err(Store* s, char* err, int n) {
  if (err && n > 0) { snprintf(err, n, "%s", s ? s->err.c_str() : "null store"); }
}

}  // namespace

extern "C" {

void* h5s_open(const char* path, int create, char* err, int errlen) {
  Store* s = new Store();
  if (!s->open(path, create != 0)) { copy_err(s, err, errlen); if (s->fd >= 0) ::close(s->fd); delete s; return nullptr; }
  return s;
}

int h5s_flush(void* h) { Store* s = (Store*)h; std::lock_guard<std::mutex> lk(s->mu); return s->flush() ? 0 : -1; }

int h5s_close(void* h) {
  Store* s = (Store*)h;
  int rc = 0;
  { std::lock_guard<std::mutex> lk(s->mu); if (!s->flush()) rc = -1; ::close(s->fd); }
  delete s;
  return rc;
}

const char* h5s_error(void* h) { return ((Store*)h)->err.c_str(); }

// values: rows*cols float16 (raw 16-bit), indices: rows*cols uint32 or null. Compression runs outside the lock.
int h5s_put(void* h, long long id, const void* values_f16, const void* indices_u32, long long rows, long long cols,
            const char* sha, const char* sample, int level) {
  Store* s = (Store*)h;
  if (rows < 0 || cols <= 0 || !values_f16) return -1;
  // level: deflate level in the low byte; bit 8 set = byte-shuffle before deflate
  const bool shuf = (level & 0x100) != 0;
  level &= 0xff;
  std::vector<uint8_t> cv, ci, tmp;
  const size_t n = (size_t)rows * cols;
  if (shuf) {
    shuffle_bytes((const uint8_t*)values_f16, n, 2, tmp);
    if (!deflate_buf(tmp.data(), n * 2, level, cv)) return -1;
    if (indices_u32) {
      shuffle_bytes((const uint8_t*)indices_u32, n, 4, tmp);
      if (!deflate_buf(tmp.data(), n * 4, level, ci)) return -1;
    }
  } else {
    if (!deflate_buf(values_f16, n * 2, level, cv)) return -1;
    if (indices_u32 && !deflate_buf(indices_u32, n * 4, level, ci)) return -1;
  }
  std::lock_guard<std::mutex> lk(s->mu);
  uint64_t dh = s->write_dataset((uint64_t)rows, (uint64_t)cols, 2, true, cv, shuf, level);
  if (dh == UNDEF) return -1;
  uint64_t ih = UNDEF;
  if (indices_u32) {
    ih = s->write_dataset((uint64_t)rows, (uint64_t)cols, 4, false, ci, shuf, level);
    if (ih == UNDEF) return -1;
  }
  return s->put_group(convo_name(id), dh, ih, sha ? sha : "", sample ? sample : "") ? 0 : -1;
}

int h5s_has(void* h, long long id) {
  Store* s = (Store*)h; std::lock_guard<std::mutex> lk(s->mu);
  return s->links.count(convo_name(id)) ? 1 : 0;
}

long long h5s_count(void* h) {
  Store* s = (Store*)h; std::lock_guard<std::mutex> lk(s->mu);
  long long n = 0;
  for (auto& kv : s->links) if (kv.first.rfind("convo_", 0) == 0) ++n;
  return n;
}

long long h5s_list_ids(void* h, long long* out, long long cap) {
  Store* s = (Store*)h; std::lock_guard<std::mutex> lk(s->mu);
  long long n = 0;
  for (auto& kv : s->links) {
    if (kv.first.rfind("convo_", 0) != 0) continue;
    const char* p = kv.first.c_str() + 6;
    char* end = nullptr;
    long long id = strtoll(p, &end, 10);
    if (end == p) continue;
    if (n < cap) out[n] = id;
    ++n;
  }
  return n;
}

// shape query: returns 0 and fills rows/cols/has_indices, or -1
int h5s_shape(void* h, long long id, long long* rows, long long* cols, int* has_indices) {
  Store* s = (Store*)h; std::lock_guard<std::mutex> lk(s->mu);
  auto it = s->links.find(convo_name(id));
  if (it == s->links.end()) { s->err = "Convo ID " + std::to_string(id) + " not found in dataset."; return -1; }
  std::vector<Store::ParsedMsg> ms;
  std::map<std::string, uint64_t> sub;
  if (!s->read_header(it->second, ms) || !s->read_group_links(ms, sub)) return -1;
  auto d = sub.find("distributions");
  if (d == sub.end()) { s->err = "Convo ID " + std::to_string(id) + " has no distributions in dataset."; return -1; }
  std::vector<Store::ParsedMsg> dm;
  if (!s->read_header(d->second, dm)) return -1;
  std::vector<uint64_t> dims;
  for (auto& m : dm)
    if (m.type == 0x0001 && m.data.size() >= 8) {
      int ver = m.data[0], rank = m.data[1];
      size_t p = ver == 1 ? 8 : 4;
      for (int i = 0; i < rank && p + 8 <= m.data.size(); ++i, p += 8) dims.push_back(rd64(&m.data[p]));
    }
  if (dims.empty()) return -1;
  *rows = (long long)dims[0];
  long long c = 1;
  for (size_t i = 1; i < dims.size(); ++i) c *= (long long)dims[i];
  *cols = c;
  *has_indices = sub.count("indices") ? 1 : 0;
  return 0;
}

// raw read: values as float16 bits (rows*cols*2 bytes), indices as uint32 (may be null)
int h5s_get(void* h, long long id, void* values_f16, void* indices_u32) {
  Store* s = (Store*)h;
  std::map<std::string, uint64_t> sub;
  {
    std::lock_guard<std::mutex> lk(s->mu);
    auto it = s->links.find(convo_name(id));
    if (it == s->links.end()) { s->err = "Convo ID " + std::to_string(id) + " not found in dataset."; return -1; }
    std::vector<Store::ParsedMsg> ms;
    if (!s->read_header(it->second, ms) || !s->read_group_links(ms, sub)) return -1;
  }
  auto d = sub.find("distributions");
  if (d == sub.end()) return -1;
  std::vector<uint8_t> raw;
  DatasetInfo info;
  if (!s->read_dataset(d->second, raw, info)) return -1;
  if (info.elem == 2) memcpy(values_f16, raw.data(), raw.size());
  else if (info.elem == 4) {  // float32 on disk: narrow is not needed by this project; reject clearly
    s->err = "distributions stored as 32-bit values are not supported"; return -1;
  }
  auto ix = sub.find("indices");
  if (ix != sub.end() && indices_u32) {
    std::vector<uint8_t> iraw; DatasetInfo ii;
    if (!s->read_dataset(ix->second, iraw, ii)) return -1;
    if (ii.elem == 4) memcpy(indices_u32, iraw.data(), iraw.size());
    else if (ii.elem == 8) { uint32_t* o = (uint32_t*)indices_u32; for (size_t i = 0; i < iraw.size() / 8; ++i) o[i] = (uint32_t)rd64(&iraw[i * 8]); }
    else { s->err = "unsupported index width"; return -1; }
  }
  return 0;
}

// string attribute of a conversation group (id >= 0) or of the root (id < 0). Returns length or -1 if absent.
long long h5s_get_attr_str(void* h, long long id, const char* name, char* out, long long cap) {
  Store* s = (Store*)h; std::lock_guard<std::mutex> lk(s->mu);
  std::string v;
  if (id < 0) {
    auto it = s->root_str_attrs.find(name);
    if (it == s->root_str_attrs.end()) return -1;
    v = it->second;
  } else {
    auto it = s->links.find(convo_name(id));
    if (it == s->links.end()) return -1;
    std::map<std::string, std::string> strs; std::map<std::string, int64_t> ints;
    if (!s->read_attrs(it->second, strs, ints)) return -1;
    auto a = strs.find(name);
    if (a == strs.end()) return -1;
    v = a->second;
  }
  if (out && cap > 0) { size_t n = std::min<size_t>(v.size(), (size_t)cap - 1); memcpy(out, v.data(), n); out[n] = 0; }
  return (long long)v.size();
}

int h5s_set_root_attr_str(void* h, const char* name, const char* value) {
  Store* s = (Store*)h; std::lock_guard<std::mutex> lk(s->mu);
  if (value) s->root_str_attrs[name] = value; else s->root_str_attrs.erase(name);
  s->dirty = true;
  return 0;
}
int h5s_get_root_attr_int(void* h, const char* name, long long* out) {
  Store* s = (Store*)h; std::lock_guard<std::mutex> lk(s->mu);
  auto it = s->root_int_attrs.find(name);
  if (it == s->root_int_attrs.end()) return -1;
  *out = it->second;
  return 0;
}
int h5s_set_root_attr_int(void* h, const char* name, long long value, int remove) {
  Store* s = (Store*)h; std::lock_guard<std::mutex> lk(s->mu);
  if (remove) s->root_int_attrs.erase(name); else s->root_int_attrs[name] = value;
  s->dirty = true;
  return 0;
}

int h5s_delete(void* h, long long id) {
  Store* s = (Store*)h; std::lock_guard<std::mutex> lk(s->mu);
  std::string n = convo_name(id);
  s->group_cache.erase(n);
  s->dirty = true;
  return s->links.erase(n) ? 0 : -1;
}

// rename map applied atomically (two-phase, so that swaps and chains work)
int h5s_rename_many(void* h, const long long* old_ids, const long long* new_ids, long long n) {
  Store* s = (Store*)h; std::lock_guard<std::mutex> lk(s->mu);
  std::vector<std::pair<std::string, uint64_t>> moved;
  std::vector<std::pair<std::string, std::pair<uint64_t, uint64_t>>> moved_cache;
  for (long long i = 0; i < n; ++i) {
    std::string o = convo_name(old_ids[i]);
    auto it = s->links.find(o);
    if (it == s->links.end()) { s->err = "rename: " + o + " not found"; return -1; }
    moved.push_back({convo_name(new_ids[i]), it->second});
    auto c = s->group_cache.find(o);
    if (c != s->group_cache.end()) { moved_cache.push_back({convo_name(new_ids[i]), c->second}); s->group_cache.erase(c); }
    s->links.erase(it);
  }
  for (auto& m : moved) s->links[m.first] = m.second;
  for (auto& m : moved_cache) s->group_cache[m.first] = m.second;
  s->dirty = true;
  return 0;
}

// rewrite the group's header with a new content_sha (datasets are reused)
int h5s_update_sha(void* h, long long id, const char* sha) {
  Store* s = (Store*)h; std::lock_guard<std::mutex> lk(s->mu);
  std::string n = convo_name(id);
  auto it = s->links.find(n);
  if (it == s->links.end()) return -1;
  std::vector<Store::ParsedMsg> ms;
  std::map<std::string, uint64_t> sub;
  if (!s->read_header(it->second, ms) || !s->read_group_links(ms, sub)) return -1;
  std::map<std::string, std::string> strs; std::map<std::string, int64_t> ints;
  if (!s->read_attrs(it->second, strs, ints)) return -1;
  auto d = sub.find("distributions");
  if (d == sub.end()) return -1;
  uint64_t ih = sub.count("indices") ? sub["indices"] : UNDEF;
  return s->put_group(n, d->second, ih, sha, strs.count("sample") ? strs["sample"] : "") ? 0 : -1;
}

long long h5s_file_bytes(void* h) { Store* s = (Store*)h; std::lock_guard<std::mutex> lk(s->mu); return (long long)s->eof; }

// Copies every live object into a fresh file (drops dead space left by deletes / replacements).
int h5s_repack(void* h, const char* dst_path) {
  Store* s = (Store*)h;
  char err[256];
  void* d = h5s_open(dst_path, 1, err, sizeof(err));
  if (!d) { s->err = err; return -1; }
  std::vector<long long> ids((size_t)h5s_count(h));
  long long n = h5s_list_ids(h, ids.data(), (long long)ids.size());
  for (long long i = 0; i < n; ++i) {
    long long rows, cols; int has_idx;
    if (h5s_shape(h, ids[i], &rows, &cols, &has_idx)) { h5s_close(d); return -1; }
    std::vector<uint16_t> v((size_t)rows * cols);
    std::vector<uint32_t> ix(has_idx ? (size_t)rows * cols : 0);
    if (h5s_get(h, ids[i], v.data(), has_idx ? ix.data() : nullptr)) { h5s_close(d); return -1; }
    std::string sha(h5s_get_attr_str(h, ids[i], "content_sha", nullptr, 0) + 1, 0), smp(h5s_get_attr_str(h, ids[i], "sample", nullptr, 0) + 1, 0);
    h5s_get_attr_str(h, ids[i], "content_sha", &sha[0], (long long)sha.size());
    h5s_get_attr_str(h, ids[i], "sample", &smp[0], (long long)smp.size());
    if (h5s_put(d, ids[i], v.data(), has_idx ? (const void*)ix.data() : nullptr, rows, cols, sha.c_str(), smp.c_str(), 6)) { h5s_close(d); return -1; }
  }
  {
    std::lock_guard<std::mutex> lk(s->mu);
    Store* ds = (Store*)d;
    ds->root_str_attrs = s->root_str_attrs;
    ds->root_int_attrs = s->root_int_attrs;
    ds->dirty = true;
  }
  return h5s_close(d);
}

}  // extern "C"
