// The host side of the paged cache in C++: the pool of pages of one group of layers and the cache
// manager above it (block tables per request and group, state slots, prefix sharing through chained
// content hashes, windows that give pages back).  Plain C++17 with a C interface; no Python, no CUDA.
//
// Semantics of the pool follow the reference's BlockPool (crates/rllm-cache/src/block_pool.rs:128-406):
// a page is handed out with reference count 1; free decrements and at 0 the page joins the free list
// keeping its hash, so that a later request with the same prefix can revive it (:247-261, :307-348);
// allocate prefers free pages without a hash and only then evicts the least recently freed hashed page,
// dropping its hash (:198-241).  Freeing a page that is not held is an error here (the reference ignores
// it).  There is no reserved null page: "no page" is -1 in a block table.
//
// The manager follows KVCacheManager (crates/rllm-cache/src/manager.rs:34-269): allocation is all or
// nothing (:132-166), block tables only grow (:162-163), full pages are shared through chained hashes
// h_k = SHA-256(h_{k-1} | tokens of page k as little-endian int64 | salt), cut to 16 bytes
// (crates/rllm-cache/src/prefix.rs:43-71; lookup manager.rs:80-121, registration after the compute
// :184-210).  Unlike it, a lookup takes no references until the request is admitted, pages are hashed only
// after their keys exist, and a prompt that is cached completely still computes its last page.
//
// Return codes of the C interface: >= 0 a result; -1 "none" (no page, no capacity); RC_* below errors.
#include <array>
#include <cstdint>
#include <cstring>
#include <list>
#include <string>
#include <unordered_map>
#include <vector>

#define RC_NOT_HELD (-2)       // a page is freed, shared or registered but not held
#define RC_BUSY (-3)           // reset of the prefix cache while hashed pages are held
#define RC_UNKNOWN_REQ (-4)
#define RC_DUPLICATE_REQ (-5)
#define RC_BADARG (-6)
#define RC_CHECK_FAILED (-7)

namespace {

using Hash16 = std::array<uint8_t, 16>;
struct Hash16Hasher {
  size_t operator()(const Hash16& h) const { size_t v; std::memcpy(&v, h.data(), sizeof v); return v; }
};

// --- SHA-256 (FIPS 180-4) ---------------------------------------------------------------------
struct Sha256 {
  uint32_t s[8];
  uint8_t buf[64];
  uint64_t len = 0;
  size_t fill = 0;
  Sha256() {
    static const uint32_t init[8] = {0x6a09e667u, 0xbb67ae85u, 0x3c6ef372u, 0xa54ff53au,
                                     0x510e527fu, 0x9b05688cu, 0x1f83d9abu, 0x5be0cd19u};
    std::memcpy(s, init, sizeof s);
  }
  static uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
  void block(const uint8_t* p) {
    static const uint32_t K[64] = {
        0x428a2f98u, 0x71374491u, 0xb5c0fbcfu, 0xe9b5dba5u, 0x3956c25bu, 0x59f111f1u, 0x923f82a4u, 0xab1c5ed5u,
        0xd807aa98u, 0x12835b01u, 0x243185beu, 0x550c7dc3u, 0x72be5d74u, 0x80deb1feu, 0x9bdc06a7u, 0xc19bf174u,
        0xe49b69c1u, 0xefbe4786u, 0x0fc19dc6u, 0x240ca1ccu, 0x2de92c6fu, 0x4a7484aau, 0x5cb0a9dcu, 0x76f988dau,
        0x983e5152u, 0xa831c66du, 0xb00327c8u, 0xbf597fc7u, 0xc6e00bf3u, 0xd5a79147u, 0x06ca6351u, 0x14292967u,
        0x27b70a85u, 0x2e1b2138u, 0x4d2c6dfcu, 0x53380d13u, 0x650a7354u, 0x766a0abbu, 0x81c2c92eu, 0x92722c85u,
        0xa2bfe8a1u, 0xa81a664bu, 0xc24b8b70u, 0xc76c51a3u, 0xd192e819u, 0xd6990624u, 0xf40e3585u, 0x106aa070u,
        0x19a4c116u, 0x1e376c08u, 0x2748774cu, 0x34b0bcb5u, 0x391c0cb3u, 0x4ed8aa4au, 0x5b9cca4fu, 0x682e6ff3u,
        0x748f82eeu, 0x78a5636fu, 0x84c87814u, 0x8cc70208u, 0x90befffau, 0xa4506cebu, 0xbef9a3f7u, 0xc67178f2u};
    uint32_t w[64];
    for (int i = 0; i < 16; ++i)
      w[i] = (uint32_t)p[4 * i] << 24 | (uint32_t)p[4 * i + 1] << 16 | (uint32_t)p[4 * i + 2] << 8 | p[4 * i + 3];
    for (int i = 16; i < 64; ++i) {
      const uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
      const uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
      w[i] = w[i - 16] + s0 + w[i - 7] + s1;
    }
    uint32_t a = s[0], b = s[1], c = s[2], d = s[3], e = s[4], f = s[5], g = s[6], h = s[7];
    for (int i = 0; i < 64; ++i) {
      const uint32_t S1 = rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25), ch = (e & f) ^ (~e & g);
      const uint32_t t1 = h + S1 + ch + K[i] + w[i];
      const uint32_t S0 = rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22), mj = (a & b) ^ (a & c) ^ (b & c);
      const uint32_t t2 = S0 + mj;
      h = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
    }
    s[0] += a; s[1] += b; s[2] += c; s[3] += d; s[4] += e; s[5] += f; s[6] += g; s[7] += h;
  }
  void update(const void* data, size_t n) {
    const uint8_t* p = (const uint8_t*)data;
    len += n;
    while (n) {
      const size_t take = n < 64 - fill ? n : 64 - fill;
      std::memcpy(buf + fill, p, take);
      fill += take; p += take; n -= take;
      if (fill == 64) { block(buf); fill = 0; }
    }
  }
  Hash16 digest16() {
    const uint64_t bits = len * 8;
    const uint8_t one = 0x80, zero = 0;
    update(&one, 1);
    while (fill != 56) update(&zero, 1);
    uint8_t lenb[8];
    for (int i = 0; i < 8; ++i) lenb[i] = (uint8_t)(bits >> (56 - 8 * i));
    update(lenb, 8);
    Hash16 out;
    for (int i = 0; i < 4; ++i) {
      out[4 * i] = (uint8_t)(s[i] >> 24); out[4 * i + 1] = (uint8_t)(s[i] >> 16);
      out[4 * i + 2] = (uint8_t)(s[i] >> 8); out[4 * i + 3] = (uint8_t)s[i];
    }
    return out;
  }
};

// chained hashes of the full pages `start` .. of tokens; parent empty (has_parent false) for page 0
void chain_hashes(const int64_t* tokens, long long n, int page_size, const uint8_t* salt, int salt_len, int start,
                  bool has_parent, Hash16 parent, std::vector<Hash16>* out) {
  for (long long k = start; k < n / page_size; ++k) {
    Sha256 h;
    if (has_parent) h.update(parent.data(), 16);
    // little-endian int64 tokens: the host is little-endian (x86-64, aarch64)
    h.update(tokens + k * page_size, (size_t)page_size * 8);
    if (salt_len > 0) h.update(salt, (size_t)salt_len);
    parent = h.digest16();
    has_parent = true;
    out->push_back(parent);
  }
}

// --- the pool ---------------------------------------------------------------------------------
struct Pool {
  int n;
  std::vector<int> ref;
  std::vector<Hash16> hash;
  std::vector<char> has_hash;
  std::unordered_map<Hash16, int, Hash16Hasher> page_of;
  std::vector<int> free_plain;                 // free pages without a hash: last in, first out
  std::list<int> free_cached;                  // free pages with findable content, least recently freed first
  std::vector<std::list<int>::iterator> where; // position in free_cached
  std::vector<char> in_cached;

  explicit Pool(int num_pages)
      : n(num_pages), ref(num_pages, 0), hash(num_pages), has_hash(num_pages, 0), where(num_pages),
        in_cached(num_pages, 0) {
    for (int p = num_pages - 1; p >= 0; --p) free_plain.push_back(p);
  }
  int num_free() const { return (int)(free_plain.size() + free_cached.size()); }
  void drop_hash(int page) {
    if (has_hash[page]) { page_of.erase(hash[page]); has_hash[page] = 0; }
  }
  int allocate() {
    int page;
    if (!free_plain.empty()) {
      page = free_plain.back();
      free_plain.pop_back();
    } else if (!free_cached.empty()) {
      page = free_cached.front();
      free_cached.pop_front();
      in_cached[page] = 0;
      drop_hash(page);
    } else {
      return -1;
    }
    ref[page] = 1;
    return page;
  }
  int incref(int page) {
    if (page < 0 || page >= n || ref[page] < 1) return RC_NOT_HELD;
    ++ref[page];
    return 0;
  }
  int release(int page) {
    if (page < 0 || page >= n || ref[page] < 1) return RC_NOT_HELD;
    if (--ref[page] == 0) {
      if (has_hash[page]) {
        free_cached.push_back(page);
        where[page] = std::prev(free_cached.end());
        in_cached[page] = 1;
      } else {
        free_plain.push_back(page);
      }
    }
    return 0;
  }
  // Copy-on-write bookkeeping (block_pool.rs:292-302): a page held by one owner is returned as it is; a shared
  // page loses this owner's reference and a fresh page is returned, into which the caller copies the data.
  int copy_on_write(int page) {
    if (page < 0 || page >= n || ref[page] < 1) return RC_NOT_HELD;
    if (ref[page] == 1) return page;
    const int fresh = allocate();
    if (fresh < 0) return -1;
    --ref[page];
    return fresh;
  }
  int reg(int page, const Hash16& h) {
    if (page < 0 || page >= n || ref[page] < 1) return RC_NOT_HELD;
    if (has_hash[page] || page_of.count(h)) return 0;   // already findable (or the same content lives elsewhere)
    hash[page] = h;
    has_hash[page] = 1;
    page_of[h] = page;
    return 0;
  }
  int peek(const Hash16& h) const {
    auto it = page_of.find(h);
    return it == page_of.end() ? -1 : it->second;
  }
  int acquire_cached(const Hash16& h) {
    auto it = page_of.find(h);
    if (it == page_of.end()) return -1;
    const int page = it->second;
    if (ref[page] == 0) {
      free_cached.erase(where[page]);
      in_cached[page] = 0;
    }
    ++ref[page];
    return page;
  }
  int reset_prefix_cache() {
    for (auto& kv : page_of)
      if (ref[kv.second] > 0) return RC_BUSY;
    for (int page : free_cached) { free_plain.push_back(page); in_cached[page] = 0; }
    free_cached.clear();
    for (auto& kv : page_of) has_hash[kv.second] = 0;
    page_of.clear();
    return 0;
  }
  // invariants: no page on the free lists twice, counts and lists agree, hashes consistent
  int check(std::string* why) const {
    std::vector<int> seen(n, 0);
    for (int p : free_plain) { if (++seen[p] > 1) { *why = "a page is on the free list twice"; return RC_CHECK_FAILED; } if (has_hash[p]) { *why = "a plain free page has a hash"; return RC_CHECK_FAILED; } }
    for (int p : free_cached) { if (++seen[p] > 1) { *why = "a page is on the free list twice"; return RC_CHECK_FAILED; } if (!has_hash[p]) { *why = "a cached free page has no hash"; return RC_CHECK_FAILED; } }
    for (int p = 0; p < n; ++p)
      if ((ref[p] == 0) != (seen[p] == 1)) { *why = "page " + std::to_string(p) + ": count and free list disagree"; return RC_CHECK_FAILED; }
    for (auto& kv : page_of)
      if (!has_hash[kv.second] || hash[kv.second] != kv.first) { *why = "hash table and pages disagree"; return RC_CHECK_FAILED; }
    return 0;
  }
};

// --- the manager --------------------------------------------------------------------------------
struct Req {
  int slot;
  std::vector<std::vector<int>> tables;     // per group (empty for groups without pages)
  std::vector<int> released;                // leading pages given back (windows)
  std::vector<Hash16> hashes;               // content hashes of this request's full pages
  int registered = 0;                       // pages already made findable
};

struct Manager {
  int num_groups, page_size, max_seqs;
  std::vector<int> kind;                    // 0: pages of keys and values, 1: state of fixed size
  std::vector<int> window;                  // per group; -1: all keys
  std::vector<int> paged;                   // group indices with pages
  std::vector<Pool*> pools;                 // per group (null for state groups)
  std::unordered_map<int64_t, Req> reqs;
  std::vector<int> free_slots, fresh_slots;
  bool prefix_caching;

  ~Manager() { for (Pool* p : pools) delete p; }
  Req* find(int64_t id) { auto it = reqs.find(id); return it == reqs.end() ? nullptr : &it->second; }
  int first_needed_page(int g, long long first_query_pos) const {
    if (window[g] < 0) return 0;
    const long long lo = first_query_pos - window[g] + 1;
    return (int)((lo > 0 ? lo : 0) / page_size);
  }
  int release_behind_window(Req* r, long long first_query_pos) {
    int n = 0;
    for (int g : paged) {
      int upto = first_needed_page(g, first_query_pos);
      if (upto > (int)r->tables[g].size()) upto = (int)r->tables[g].size();
      for (int k = r->released[g]; k < upto; ++k)
        if (r->tables[g][k] >= 0) { pools[g]->release(r->tables[g][k]); r->tables[g][k] = -1; ++n; }
      if (upto > r->released[g]) r->released[g] = upto;
    }
    return n;
  }
  // How many leading pages with these hashes a new request can take over: the largest k such that every
  // group has, findable, all pages below k that a query at position k * page_size can still see (all of
  // them where every key is kept; those that reach into the window elsewhere).
  long long shareable_pages(const std::vector<Hash16>& hs) const {
    long long k = (long long)hs.size();
    for (int g : paged) {
      if (window[g] >= 0) continue;
      long long have = 0;
      while (have < k && pools[g]->peek(hs[have]) >= 0) ++have;
      k = have;
    }
    for (; k > 0; --k) {
      bool ok = true;
      for (int g : paged) {
        if (window[g] < 0) continue;
        for (long long j = first_needed_page(g, k * page_size); j < k && ok; ++j) ok = pools[g]->peek(hs[j]) >= 0;
        if (!ok) break;
      }
      if (ok) break;
    }
    return k;
  }
  int pages_needed(const Req* r, int g, long long first_query_pos, long long num_tokens) const {
    const long long want = (num_tokens + page_size - 1) / page_size;
    long long first = first_needed_page(g, first_query_pos);
    if ((long long)r->tables[g].size() > first) first = (long long)r->tables[g].size();
    return (int)(want > first ? want - first : 0);
  }
};

Manager* M(void* h) { return (Manager*)h; }
Pool* P(void* h) { return (Pool*)h; }
Hash16 as_hash(const uint8_t* p) { Hash16 h; std::memcpy(h.data(), p, 16); return h; }

}  // namespace

extern "C" {
#define API __attribute__((visibility("default")))

// ---- hashes ----
// out: 16 bytes per full page from page `start` on; returns their number.  parent: 16 bytes or null.
API long long rllm_page_hashes(const int64_t* tokens, long long n, int page_size, const uint8_t* salt, int salt_len,
                               int start, const uint8_t* parent, uint8_t* out, long long cap) {
  if (page_size < 1 || n < 0 || start < 0) return RC_BADARG;
  std::vector<Hash16> hs;
  chain_hashes(tokens, n, page_size, salt, salt_len, start, parent != nullptr, parent ? as_hash(parent) : Hash16(), &hs);
  if ((long long)hs.size() > cap) return RC_BADARG;
  for (size_t i = 0; i < hs.size(); ++i) std::memcpy(out + 16 * i, hs[i].data(), 16);
  return (long long)hs.size();
}

// ---- pool ----
API void* rllm_pool_new(int num_pages) { return num_pages < 1 ? nullptr : new Pool(num_pages); }
API void rllm_pool_delete(void* h) { delete P(h); }
API int rllm_pool_num_pages(void* h) { return P(h)->n; }
API int rllm_pool_num_free(void* h) { return P(h)->num_free(); }
API int rllm_pool_num_cached(void* h) { return (int)P(h)->page_of.size(); }
API int rllm_pool_allocate(void* h) { return P(h)->allocate(); }
API int rllm_pool_incref(void* h, int page) { return P(h)->incref(page); }
API int rllm_pool_free(void* h, int page) { return P(h)->release(page); }
API int rllm_pool_refcount(void* h, int page) { return page < 0 || page >= P(h)->n ? RC_BADARG : P(h)->ref[page]; }
API int rllm_pool_copy_on_write(void* h, int page) { return P(h)->copy_on_write(page); }
API int rllm_pool_register(void* h, int page, const uint8_t* hash) { return P(h)->reg(page, as_hash(hash)); }
API int rllm_pool_peek(void* h, const uint8_t* hash) { return P(h)->peek(as_hash(hash)); }
API int rllm_pool_acquire_cached(void* h, const uint8_t* hash) { return P(h)->acquire_cached(as_hash(hash)); }
API int rllm_pool_reset_prefix_cache(void* h) { return P(h)->reset_prefix_cache(); }
API int rllm_pool_check(void* h, char* why, int cap) {
  std::string s;
  const int rc = P(h)->check(&s);
  if (why && cap > 0) { std::strncpy(why, s.c_str(), cap - 1); why[cap - 1] = 0; }
  return rc;
}

// ---- manager ----
// kinds[g]: 0 pages, 1 state; windows[g]: keys a query sees, or -1 for all; num_pages[g]: pages of a paged group
API void* rllm_cache_new(int num_groups, const int* kinds, const int* windows, const int* num_pages, int page_size,
                         int max_seqs, int enable_prefix_caching) {
  if (num_groups < 0 || page_size < 1 || max_seqs < 1) return nullptr;
  Manager* m = new Manager();
  m->num_groups = num_groups; m->page_size = page_size; m->max_seqs = max_seqs;
  bool stateful = false;
  for (int g = 0; g < num_groups; ++g) {
    m->kind.push_back(kinds[g]);
    m->window.push_back(windows[g]);
    if (kinds[g] == 0) {
      if (num_pages[g] < 1) { delete m; return nullptr; }
      m->paged.push_back(g);
      m->pools.push_back(new Pool(num_pages[g]));
    } else {
      stateful = true;
      m->pools.push_back(nullptr);
    }
  }
  for (int s = max_seqs - 1; s >= 0; --s) m->free_slots.push_back(s);
  // State of fixed size cannot be taken over from pages: with such a group every request computes its own.
  m->prefix_caching = enable_prefix_caching && !stateful && !m->paged.empty();
  return m;
}
API void rllm_cache_delete(void* h) { delete M(h); }
API int rllm_cache_prefix_caching(void* h) { return M(h)->prefix_caching ? 1 : 0; }
API void* rllm_cache_pool(void* h, int g) { return g < 0 || g >= M(h)->num_groups ? nullptr : M(h)->pools[g]; }
API int rllm_cache_num_requests(void* h) { return (int)M(h)->reqs.size(); }
API int rllm_cache_num_free_slots(void* h) { return (int)M(h)->free_slots.size(); }
API int rllm_cache_has(void* h, int64_t id) { return M(h)->find(id) ? 1 : 0; }

API int rllm_cache_admit(void* h, int64_t id) {
  Manager* m = M(h);
  if (m->find(id)) return RC_DUPLICATE_REQ;
  if (m->free_slots.empty()) return -1;
  Req r;
  r.slot = m->free_slots.back();
  m->free_slots.pop_back();
  r.tables.resize(m->num_groups);
  r.released.assign(m->num_groups, 0);
  m->fresh_slots.push_back(r.slot);
  const int slot = r.slot;
  m->reqs.emplace(id, std::move(r));
  return slot;
}
// slots handed out since the last call (their state must be zeroed before the next step)
API int rllm_cache_take_fresh_slots(void* h, int* out, int cap) {
  Manager* m = M(h);
  const int n = (int)m->fresh_slots.size();
  if (n > cap) return RC_BADARG;
  for (int i = 0; i < n; ++i) out[i] = m->fresh_slots[i];
  m->fresh_slots.clear();
  return n;
}
API int rllm_cache_num_fresh_slots(void* h) { return (int)M(h)->fresh_slots.size(); }
API int rllm_cache_free(void* h, int64_t id) {
  Manager* m = M(h);
  auto it = m->reqs.find(id);
  if (it == m->reqs.end()) return 0;
  Req& r = it->second;
  // Last page first (the reference frees in table order, crates/rllm-cache/src/manager.rs:169-177): of a
  // request's findable pages the last are then evicted first, and a prefix stays findable as long as its
  // first pages are; and pages without a hash come back in rising order, so that the next request's
  // pages follow one another in the cache.
  for (int g : m->paged)
    for (auto it = r.tables[g].rbegin(); it != r.tables[g].rend(); ++it)
      if (*it >= 0) m->pools[g]->release(*it);
  m->free_slots.push_back(r.slot);
  for (size_t i = 0; i < m->fresh_slots.size(); ++i)
    if (m->fresh_slots[i] == r.slot) { m->fresh_slots.erase(m->fresh_slots.begin() + i); break; }
  m->reqs.erase(it);
  return 0;
}
// A child request that starts as a copy of the first num_tokens tokens of a parent
// (crates/rllm-cache/src/manager.rs:220-245 shares every page and leaves the copy to the first write; here the
// one page that both would write, the partly filled last one, is made the child's own at once).  The child
// gets a slot of its own, shares the parent's full pages by reference count, and gets a fresh page for the
// partly filled one in every paged group.  copies: triples (group, page of the parent, page of the child)
// whose data the caller must copy, and the pair of state slots is (slot of parent, returned slot).
// Returns the child's slot; -1 if a slot or a page is missing (nothing taken); RC_* on errors.
API int rllm_cache_fork(void* h, int64_t parent_id, int64_t child_id, long long num_tokens, int* copies, int cap,
                        int* num_copies) {
  Manager* m = M(h);
  if (m->find(child_id)) return RC_DUPLICATE_REQ;
  Req* p = m->find(parent_id);
  if (!p) return RC_UNKNOWN_REQ;
  if (num_tokens < 0 || !num_copies) return RC_BADARG;
  const long long want = (num_tokens + m->page_size - 1) / m->page_size;
  const bool partial = num_tokens % m->page_size != 0;
  int n_copy = 0;
  for (int g : m->paged) {
    if ((long long)p->tables[g].size() < want) return RC_NOT_HELD;       // the parent does not hold that much
    // a window may have passed pages that the child's next query (at position num_tokens) would still see
    for (long long k = m->first_needed_page(g, num_tokens); k < want; ++k)
      if (p->tables[g][k] < 0) return RC_NOT_HELD;
    if (partial && p->tables[g][want - 1] >= 0) {
      if (m->pools[g]->num_free() < 1) return -1;
      ++n_copy;
    }
  }
  if (m->free_slots.empty()) return -1;
  if (3 * n_copy > cap) return RC_BADARG;
  Req c;
  c.slot = m->free_slots.back();
  m->free_slots.pop_back();
  c.tables.resize(m->num_groups);
  c.released.assign(m->num_groups, 0);
  int k = 0;
  for (int g : m->paged) {
    c.tables[g].assign(p->tables[g].begin(), p->tables[g].begin() + want);
    c.released[g] = p->released[g] < (int)want ? p->released[g] : (int)want;
    for (int page : c.tables[g])
      if (page >= 0) m->pools[g]->incref(page);
    if (partial && c.tables[g][want - 1] >= 0) {
      const int shared = c.tables[g][want - 1];
      const int own = m->pools[g]->copy_on_write(shared);      // shared by two now: a fresh page comes back
      c.tables[g][want - 1] = own;
      copies[3 * k] = g; copies[3 * k + 1] = shared; copies[3 * k + 2] = own;
      ++k;
    }
  }
  const size_t full = (size_t)(num_tokens / m->page_size);
  c.hashes.assign(p->hashes.begin(), p->hashes.begin() + (p->hashes.size() < full ? p->hashes.size() : full));
  c.registered = p->registered < (int)full ? p->registered : (int)full;
  if (c.registered > (int)c.hashes.size()) c.registered = (int)c.hashes.size();
  *num_copies = k;
  const int slot = c.slot;                                       // not a fresh slot: the caller copies the state into it
  m->reqs.emplace(child_id, std::move(c));
  return slot;
}
API int rllm_cache_slot(void* h, int64_t id) {
  Req* r = M(h)->find(id);
  return r ? r->slot : RC_UNKNOWN_REQ;
}
API int rllm_cache_table_len(void* h, int64_t id, int g) {
  Req* r = M(h)->find(id);
  if (!r) return RC_UNKNOWN_REQ;
  if (g < 0 || g >= M(h)->num_groups) return RC_BADARG;
  return (int)r->tables[g].size();
}
// the first min(len, cap) entries of the table go to out, the rest of out[0..cap) is filled with -1; returns len
API int rllm_cache_table(void* h, int64_t id, int g, int* out, int cap) {
  Req* r = M(h)->find(id);
  if (!r) return RC_UNKNOWN_REQ;
  if (g < 0 || g >= M(h)->num_groups) return RC_BADARG;
  const std::vector<int>& t = r->tables[g];
  const int n = (int)t.size() < cap ? (int)t.size() : cap;
  for (int i = 0; i < n; ++i) out[i] = t[i];
  for (int i = n; i < cap; ++i) out[i] = -1;
  return (int)t.size();
}
API int rllm_cache_release_behind_window(void* h, int64_t id, long long first_query_pos) {
  Req* r = M(h)->find(id);
  return r ? M(h)->release_behind_window(r, first_query_pos) : RC_UNKNOWN_REQ;
}
API int rllm_cache_pages_needed(void* h, int64_t id, int g, long long first_query_pos, long long num_tokens) {
  Req* r = M(h)->find(id);
  if (!r) return RC_UNKNOWN_REQ;
  return M(h)->pages_needed(r, g, first_query_pos, num_tokens);
}
// pages for positions < num_tokens that queries from first_query_pos on can see, in every paged group;
// all or nothing: 1 done, 0 nothing taken
API int rllm_cache_ensure(void* h, int64_t id, long long first_query_pos, long long num_tokens) {
  Manager* m = M(h);
  Req* r = m->find(id);
  if (!r) return RC_UNKNOWN_REQ;
  m->release_behind_window(r, first_query_pos);
  for (int g : m->paged)
    if (m->pools[g]->num_free() < m->pages_needed(r, g, first_query_pos, num_tokens)) return 0;
  const long long want = (num_tokens + m->page_size - 1) / m->page_size;
  for (int g : m->paged) {
    const int first = m->first_needed_page(g, first_query_pos);
    while ((long long)r->tables[g].size() < want) {
      const int k = (int)r->tables[g].size();
      if (k < first) {            // behind the window from the start: never held
        r->tables[g].push_back(-1);
        r->released[g] = k + 1;
      } else {
        r->tables[g].push_back(m->pools[g]->allocate());
      }
    }
  }
  return 1;
}
// The largest num_tokens for which rllm_cache_ensure(id, first_query_pos, num_tokens) would succeed now.
// Gives back the pages behind the window of first_query_pos first (ensure would do the same).
API long long rllm_cache_max_tokens(void* h, int64_t id, long long first_query_pos) {
  Manager* m = M(h);
  Req* r = m->find(id);
  if (!r) return RC_UNKNOWN_REQ;
  m->release_behind_window(r, first_query_pos);
  long long best = -1;
  for (int g : m->paged) {
    long long first = m->first_needed_page(g, first_query_pos);
    if ((long long)r->tables[g].size() > first) first = (long long)r->tables[g].size();
    const long long upto = (first + m->pools[g]->num_free()) * m->page_size;
    if (best < 0 || upto < best) best = upto;
  }
  return best < 0 ? (1LL << 62) : best;
}
API int rllm_cache_fits_at_all(void* h, long long num_tokens) {
  Manager* m = M(h);
  const long long want = (num_tokens + m->page_size - 1) / m->page_size;
  for (int g : m->paged) {
    long long want_g = want;
    if (m->window[g] >= 0) {
      const long long w = (m->window[g] + m->page_size + m->page_size - 1) / m->page_size + 1;
      if (w < want_g) want_g = w;
    }
    if (want_g > m->pools[g]->n) return 0;
  }
  return 1;
}
// how many leading tokens lie in findable pages (no reference taken); a prompt cached completely reports a page less
API long long rllm_cache_match_prefix(void* h, const int64_t* tokens, long long n) {
  Manager* m = M(h);
  if (!m->prefix_caching) return 0;
  std::vector<Hash16> hs;
  chain_hashes(tokens, n, m->page_size, nullptr, 0, 0, false, Hash16(), &hs);
  if (!hs.empty() && (long long)hs.size() * m->page_size >= n) hs.pop_back();
  return m->shareable_pages(hs) * m->page_size;
}
// gives a newly admitted request the findable pages of its prefix; returns the tokens it need not compute.
// In a group that keeps a window the pages that the request's first query can no longer see are not taken
// (their table entries are -1, as if the window had passed them).
API long long rllm_cache_adopt_prefix(void* h, int64_t id, const int64_t* tokens, long long n) {
  Manager* m = M(h);
  if (!m->prefix_caching) return 0;
  Req* r = m->find(id);
  if (!r) return RC_UNKNOWN_REQ;
  for (int g : m->paged)
    if (!r->tables[g].empty()) return RC_NOT_HELD;
  const long long limit = n > 0 ? (n - 1) / m->page_size : 0;    // keep at least one token to compute
  std::vector<Hash16> hs;
  chain_hashes(tokens, limit * m->page_size, m->page_size, nullptr, 0, 0, false, Hash16(), &hs);
  const long long got = m->shareable_pages(hs);
  for (int g : m->paged) {
    const long long first = m->first_needed_page(g, got * m->page_size);
    for (long long k = 0; k < got; ++k)
      r->tables[g].push_back(k < first ? -1 : m->pools[g]->acquire_cached(hs[k]));
    r->released[g] = (int)(first < got ? first : got);
  }
  hs.resize((size_t)got);
  r->hashes = hs;
  r->registered = (int)got;
  return got * m->page_size;
}
// makes the pages findable whose keys now exist for all their tokens
API int rllm_cache_register_computed(void* h, int64_t id, const int64_t* tokens, long long n, long long num_computed) {
  Manager* m = M(h);
  if (!m->prefix_caching) return 0;
  Req* r = m->find(id);
  if (!r) return RC_UNKNOWN_REQ;
  const long long upto = num_computed < n ? num_computed : n;
  const long long full = upto / m->page_size;
  if (full > (long long)r->hashes.size()) {
    const bool has_parent = !r->hashes.empty();
    chain_hashes(tokens, full * m->page_size, m->page_size, nullptr, 0, (int)r->hashes.size(), has_parent,
                 has_parent ? r->hashes.back() : Hash16(), &r->hashes);
  }
  for (int g : m->paged)
    for (long long k = r->registered; k < full; ++k)
      if (r->tables[g][k] >= 0) m->pools[g]->reg(r->tables[g][k], r->hashes[k]);   // (-1: the window has passed it)
  if (full > r->registered) r->registered = (int)full;
  return 0;
}
// no page lost, held twice without a matching count, or freed twice; no state slot lost or held twice
API int rllm_cache_check(void* h, char* why, int cap) {
  Manager* m = M(h);
  std::string s;
  int rc = 0;
  for (int g : m->paged) {
    rc = m->pools[g]->check(&s);
    if (rc) break;
    std::vector<int> held(m->pools[g]->n, 0);
    for (auto& kv : m->reqs)
      for (int page : kv.second.tables[g])
        if (page >= 0) ++held[page];
    for (int p = 0; p < m->pools[g]->n && !rc; ++p)
      if (held[p] != m->pools[g]->ref[p]) {
        s = "group " + std::to_string(g) + " page " + std::to_string(p) + ": count " +
            std::to_string(m->pools[g]->ref[p]) + ", held by " + std::to_string(held[p]);
        rc = RC_CHECK_FAILED;
      }
    if (rc) break;
  }
  if (!rc) {
    std::vector<int> seen(m->max_seqs, 0);
    for (auto& kv : m->reqs) ++seen[kv.second.slot];
    for (int sl : m->free_slots) ++seen[sl];
    for (int i = 0; i < m->max_seqs; ++i)
      if (seen[i] != 1) { s = "a state slot is lost or held twice"; rc = RC_CHECK_FAILED; break; }
  }
  if (why && cap > 0) { std::strncpy(why, s.c_str(), cap - 1); why[cap - 1] = 0; }
  return rc;
}

// The rows of a step's block table in one call: row i of out (width entries) gets the table of request
// ids[i] in group g, -1 behind its end.  Returns 0 or RC_UNKNOWN_REQ.
API int rllm_cache_pack_tables(void* h, const int64_t* ids, int n, int g, int* out, int width) {
  Manager* m = M(h);
  if (g < 0 || g >= m->num_groups || width < 0) return RC_BADARG;
  for (int i = 0; i < n; ++i) {
    Req* r = m->find(ids[i]);
    if (!r) return RC_UNKNOWN_REQ;
    const std::vector<int>& t = r->tables[g];
    int* row = out + (size_t)i * width;
    const int k = (int)t.size() < width ? (int)t.size() : width;
    for (int j = 0; j < k; ++j) row[j] = t[j];
    for (int j = k; j < width; ++j) row[j] = -1;
  }
  return 0;
}

}  // extern "C"
