// Host-side runtime of the paged cache, in C++ behind a C interface: page pools with ownership checks, block
// tables for every layer group, request slots, window release, rewind and a full audit.  Nothing here touches
// the GPU; the Python classes in hk_b200/cache/pages.py are thin views of these objects (tables and lengths are
// read in place through numpy).
//
// Every call that can fail returns a negative code and leaves the books unchanged; hk_books_error() gives the
// message of the last failure.  Reference analogues: a slot per sequence with a fixed region
// (src/cuda/engine.zig:393-401,556-572), segments grown on demand and freed on rewind
// (src/engine/kv.zig:88-109,137-151), ContextFull / NoGpuSlot (src/engine/model.zig:298, src/cuda/engine.zig:564).
#include <stdint.h>

#include <algorithm>
#include <map>
#include <string>
#include <utility>
#include <vector>

#define HK_API extern "C" __attribute__((visibility("default")))

namespace {

enum Error {
  ERR_OUT_OF_PAGES = -1,
  ERR_TOO_MANY_REQUESTS = -2,
  ERR_CONTEXT_FULL = -3,
  ERR_CACHE = -4,        // a broken invariant or a slot that is not live
  ERR_VALUE = -5,        // an argument out of range
};

// Free list of page ids 0..n-1 with ownership checks; the page freed last is reused first.
struct Pool {
  int n = 0;
  std::vector<int> free_list;
  std::vector<uint8_t> held;
  std::string error;

  explicit Pool(int num_pages) : n(num_pages), held((size_t)num_pages, 0) {
    free_list.reserve((size_t)num_pages);
    for (int p = num_pages - 1; p >= 0; --p) free_list.push_back(p);     // take() gives 0 first
  }
  int take() {
    if (free_list.empty()) {
      error = "no free page";
      return ERR_OUT_OF_PAGES;
    }
    const int p = free_list.back();
    if (held[(size_t)p]) {
      error = "page " + std::to_string(p) + " was on the free list while held";
      return ERR_CACHE;
    }
    free_list.pop_back();
    held[(size_t)p] = 1;
    return p;
  }
  int give(int p) {
    if (p < 0 || p >= n || !held[(size_t)p]) {
      error = "page " + std::to_string(p) + " is given back but not held";
      return ERR_CACHE;
    }
    held[(size_t)p] = 0;
    free_list.push_back(p);
    return 0;
  }
};

struct Group {
  int window;                       // -1: every key stays
  Pool pool;
  std::vector<int32_t> table;       // [max_requests][max_pages], -1 = none
  std::vector<int32_t> first_page;  // lowest logical page still held
  std::vector<int32_t> n_pages;     // logical pages ever reached (held or passed)
  Group(int w, int num_pages, int max_requests, int max_pages)
      : window(w), pool(num_pages), table((size_t)max_requests * max_pages, -1), first_page((size_t)max_requests, 0),
        n_pages((size_t)max_requests, 0) {}
};

struct Books {
  int page_tokens, max_requests, max_context, max_pages;
  std::vector<Group> groups;
  std::vector<int> free_slots;
  std::vector<int64_t> length;
  std::vector<uint8_t> live;
  std::string error;

  int fail(int code, const std::string& msg) {
    error = msg;
    return code;
  }
  bool is_live(int slot) const { return slot >= 0 && slot < max_requests && live[(size_t)slot]; }
  int32_t& entry(Group& g, int slot, int i) { return g.table[(size_t)slot * max_pages + i]; }
  int pages_for(int64_t tokens) const { return (int)((tokens + page_tokens - 1) / page_tokens); }

  // Logical pages [first_page, end) of a windowed group that no later token can read: the next query sits at
  // position `cur` and reads keys from cur - window + 1 on.
  int passed_end(const Group& g, int slot, int64_t cur) const {
    if (g.window < 0) return g.first_page[(size_t)slot];
    const int64_t first_needed = std::max<int64_t>(0, cur - g.window + 1) / page_tokens;
    return (int)std::max<int64_t>(g.first_page[(size_t)slot], std::min<int64_t>(first_needed, g.n_pages[(size_t)slot]));
  }

  int release_passed(int slot) {
    if (!is_live(slot)) return fail(ERR_CACHE, "slot " + std::to_string(slot) + " is not live");
    const int64_t cur = length[(size_t)slot];
    int n = 0;
    for (Group& g : groups) {
      const int end = passed_end(g, slot, cur);
      for (int i = g.first_page[(size_t)slot]; i < end; ++i) {
        const int rc = g.pool.give(entry(g, slot, i));
        if (rc < 0) return fail(rc, g.pool.error);
        entry(g, slot, i) = -1;
        g.first_page[(size_t)slot] = i + 1;
        ++n;
      }
    }
    return n;
  }
};

}  // namespace

// ---- a pool on its own --------------------------------------------------------------------------------

HK_API void* hk_pool_create(int num_pages) { return num_pages < 1 ? nullptr : new Pool(num_pages); }
HK_API void hk_pool_destroy(void* p) { delete static_cast<Pool*>(p); }
HK_API int hk_pool_take(void* p) { return static_cast<Pool*>(p)->take(); }
HK_API int hk_pool_give(void* p, int page) { return static_cast<Pool*>(p)->give(page); }
HK_API int hk_pool_free_count(void* p) { return (int)static_cast<Pool*>(p)->free_list.size(); }
HK_API int hk_pool_num_pages(void* p) { return static_cast<Pool*>(p)->n; }
HK_API const uint8_t* hk_pool_held(void* p) { return static_cast<Pool*>(p)->held.data(); }
HK_API const char* hk_pool_error(void* p) { return static_cast<Pool*>(p)->error.c_str(); }

// ---- the books ------------------------------------------------------------------------------------------

// windows[g] < 0: the group keeps every key; else only the last windows[g] positions are ever read again.
HK_API void* hk_books_create(const int* windows, int n_groups, int page_tokens, int num_pages, int max_requests, int max_context) {
  if (page_tokens < 1 || max_requests < 1 || max_context < 1 || num_pages < 1 || n_groups < 0) return nullptr;
  Books* b = new Books();
  b->page_tokens = page_tokens;
  b->max_requests = max_requests;
  b->max_context = max_context;
  b->max_pages = (max_context + page_tokens - 1) / page_tokens;
  for (int g = 0; g < n_groups; ++g) b->groups.emplace_back(windows[g], num_pages, max_requests, b->max_pages);
  for (int s = max_requests - 1; s >= 0; --s) b->free_slots.push_back(s);
  b->length.assign((size_t)max_requests, 0);
  b->live.assign((size_t)max_requests, 0);
  return b;
}
HK_API void hk_books_destroy(void* h) { delete static_cast<Books*>(h); }
HK_API const char* hk_books_error(void* h) { return static_cast<Books*>(h)->error.c_str(); }
HK_API int hk_books_max_pages(void* h) { return static_cast<Books*>(h)->max_pages; }
HK_API int64_t* hk_books_length(void* h) { return static_cast<Books*>(h)->length.data(); }
HK_API uint8_t* hk_books_live(void* h) { return static_cast<Books*>(h)->live.data(); }
HK_API void* hk_books_pool(void* h, int g) { return &static_cast<Books*>(h)->groups[(size_t)g].pool; }
HK_API int32_t* hk_books_table(void* h, int g) { return static_cast<Books*>(h)->groups[(size_t)g].table.data(); }
HK_API int32_t* hk_books_first_page(void* h, int g) { return static_cast<Books*>(h)->groups[(size_t)g].first_page.data(); }
HK_API int32_t* hk_books_n_pages(void* h, int g) { return static_cast<Books*>(h)->groups[(size_t)g].n_pages.data(); }

HK_API int hk_books_open(void* h) {
  Books& b = *static_cast<Books*>(h);
  if (b.free_slots.empty()) return b.fail(ERR_TOO_MANY_REQUESTS, "all " + std::to_string(b.max_requests) + " request slots are in use");
  const int s = b.free_slots.back();
  b.free_slots.pop_back();
  b.live[(size_t)s] = 1;
  b.length[(size_t)s] = 0;
  for (Group& g : b.groups) g.first_page[(size_t)s] = g.n_pages[(size_t)s] = 0;
  return s;
}

HK_API int hk_books_close(void* h, int slot) {
  Books& b = *static_cast<Books*>(h);
  if (!b.is_live(slot)) return b.fail(ERR_CACHE, "slot " + std::to_string(slot) + " is not live");
  for (Group& g : b.groups) {
    for (int i = g.first_page[(size_t)slot]; i < g.n_pages[(size_t)slot]; ++i) {
      const int p = b.entry(g, slot, i);
      if (p >= 0) {
        const int rc = g.pool.give(p);
        if (rc < 0) return b.fail(rc, g.pool.error);
      }
    }
    for (int i = 0; i < g.n_pages[(size_t)slot]; ++i) b.entry(g, slot, i) = -1;
    g.first_page[(size_t)slot] = g.n_pages[(size_t)slot] = 0;
  }
  b.live[(size_t)slot] = 0;
  b.length[(size_t)slot] = 0;
  b.free_slots.push_back(slot);
  return 0;
}

// Gives back the pages of `slot` that its windows have passed; returns how many.
HK_API int hk_books_release_passed(void* h, int slot) { return static_cast<Books*>(h)->release_passed(slot); }

// For each group: the pages hk_books_release_passed(slot) would give back now.
HK_API int hk_books_pages_passed(void* h, int slot, int* out) {
  Books& b = *static_cast<Books*>(h);
  if (!b.is_live(slot)) return b.fail(ERR_CACHE, "slot " + std::to_string(slot) + " is not live");
  for (size_t g = 0; g < b.groups.size(); ++g)
    out[g] = b.passed_end(b.groups[g], slot, b.length[(size_t)slot]) - b.groups[g].first_page[(size_t)slot];
  return 0;
}

// For each group: the pages hk_books_extend(slot, n_new) would take from the pool.
HK_API int hk_books_pages_to_take(void* h, int slot, int n_new, int* out) {
  Books& b = *static_cast<Books*>(h);
  if (!b.is_live(slot)) return b.fail(ERR_CACHE, "slot " + std::to_string(slot) + " is not live");
  const int want = b.pages_for(b.length[(size_t)slot] + n_new);
  for (size_t g = 0; g < b.groups.size(); ++g) out[g] = std::max(0, want - b.groups[g].n_pages[(size_t)slot]);
  return 0;
}

HK_API void hk_books_free_pages(void* h, int* out) {
  Books& b = *static_cast<Books*>(h);
  for (size_t g = 0; g < b.groups.size(); ++g) out[g] = (int)b.groups[g].pool.free_list.size();
}

// Makes room for n_new more tokens of `slot`: gives back pages the window has passed, then takes the pages the
// new positions need - all of them or none.  Returns how many table entries changed.
HK_API int hk_books_extend(void* h, int slot, int n_new) {
  Books& b = *static_cast<Books*>(h);
  if (!b.is_live(slot)) return b.fail(ERR_CACHE, "slot " + std::to_string(slot) + " is not live");
  if (n_new < 1) return b.fail(ERR_VALUE, "extend needs at least one token");
  const int64_t cur = b.length[(size_t)slot];
  if (cur + n_new > b.max_context)
    return b.fail(ERR_CONTEXT_FULL, "request would reach " + std::to_string(cur + n_new) + " tokens; the context holds " +
                                        std::to_string(b.max_context));
  // what the window would give back counts as free for this check, but nothing is touched before the check passes
  const int want = b.pages_for(cur + n_new);
  for (Group& g : b.groups) {
    const int k = std::max(0, want - g.n_pages[(size_t)slot]);
    const int back = b.passed_end(g, slot, cur) - g.first_page[(size_t)slot];
    if (k > (int)g.pool.free_list.size() + back)
      return b.fail(ERR_OUT_OF_PAGES, std::to_string(k) + " pages needed, " + std::to_string((int)g.pool.free_list.size() + back) + " free");
  }
  int changed = b.release_passed(slot);
  if (changed < 0) return changed;
  for (Group& g : b.groups) {
    for (int i = g.n_pages[(size_t)slot]; i < want; ++i) {
      const int p = g.pool.take();
      if (p < 0) return b.fail(p, g.pool.error);         // cannot happen after the check above
      b.entry(g, slot, i) = p;
      ++changed;
    }
    g.n_pages[(size_t)slot] = std::max(g.n_pages[(size_t)slot], want);
  }
  b.length[(size_t)slot] = cur + n_new;
  return changed;
}

// Rewinds `slot` to `keep` tokens, giving back the pages above.  A windowed group cannot rewind below what it
// already gave back.
HK_API int hk_books_truncate(void* h, int slot, int keep) {
  Books& b = *static_cast<Books*>(h);
  if (!b.is_live(slot)) return b.fail(ERR_CACHE, "slot " + std::to_string(slot) + " is not live");
  if (keep < 0 || keep > b.length[(size_t)slot]) return b.fail(ERR_VALUE, "truncate keeps between 0 and the current length");
  const int keep_pages = b.pages_for(keep);
  for (Group& g : b.groups)
    if (g.window >= 0 && keep > 0 && std::max(0, keep - g.window) / b.page_tokens < g.first_page[(size_t)slot])
      return b.fail(ERR_CACHE, "cannot rewind a windowed cache below pages it has given back");
  for (Group& g : b.groups) {
    for (int i = std::max(keep_pages, (int)g.first_page[(size_t)slot]); i < g.n_pages[(size_t)slot]; ++i) {
      const int rc = g.pool.give(b.entry(g, slot, i));
      if (rc < 0) return b.fail(rc, g.pool.error);
      b.entry(g, slot, i) = -1;
    }
    g.n_pages[(size_t)slot] = std::min<int32_t>(g.n_pages[(size_t)slot], keep_pages);
    g.first_page[(size_t)slot] = std::min<int32_t>(g.first_page[(size_t)slot], keep_pages);
  }
  b.length[(size_t)slot] = keep;
  return 0;
}

// Fails if a page is lost, held twice, or free while in a table.
HK_API int hk_books_audit(void* h) {
  Books& b = *static_cast<Books*>(h);
  for (size_t gi = 0; gi < b.groups.size(); ++gi) {
    Group& g = b.groups[gi];
    std::map<int, std::pair<int, int>> seen;
    for (int s = 0; s < b.max_requests; ++s) {
      for (int i = 0; i < b.max_pages; ++i) {
        const int p = b.entry(g, s, i);
        if (p < 0) continue;
        if (!b.live[(size_t)s]) return b.fail(ERR_CACHE, "group " + std::to_string(gi) + ": dead slot " + std::to_string(s) + " still lists pages");
        auto it = seen.find(p);
        if (it != seen.end())
          return b.fail(ERR_CACHE, "group " + std::to_string(gi) + ": page " + std::to_string(p) + " is held twice ((" +
                                       std::to_string(it->second.first) + ", " + std::to_string(it->second.second) + ") and (" +
                                       std::to_string(s) + ", " + std::to_string(i) + "))");
        seen[p] = {s, i};
      }
    }
    int held = 0;
    for (int p = 0; p < g.pool.n; ++p) {
      const bool listed = seen.count(p) != 0;
      if (g.pool.held[(size_t)p] && !listed) return b.fail(ERR_CACHE, "group " + std::to_string(gi) + ": the pool holds page " + std::to_string(p) + " that no table lists");
      if (!g.pool.held[(size_t)p] && listed) return b.fail(ERR_CACHE, "group " + std::to_string(gi) + ": a table lists page " + std::to_string(p) + " that the pool does not hold");
      held += g.pool.held[(size_t)p];
    }
    if (held + (int)g.pool.free_list.size() != g.pool.n)
      return b.fail(ERR_CACHE, "group " + std::to_string(gi) + ": " + std::to_string(g.pool.n - held - (int)g.pool.free_list.size()) + " pages lost");
  }
  return 0;
}
