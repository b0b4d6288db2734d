// Paged cache manager: page pools with reference counts, one block table per
// request and cache group, and fixed-size state slots.
//
// A cache group is a set of layer caches with the same needs: all keys of a
// request (window == 0) or only the last `window` of them.  Every group has
// pages of its own.  A page id names a slot in every layer cache of its
// group, so a request has one block table per group, not per layer.
//
// Semantics follow the reference's physical pool (runtime/kv/pool.mojo:28-114:
// reference counts, a LIFO free stack whose first allocations are 0,1,2,...,
// release returns whether the page was freed) and its request views
// (runtime/kv/space.mojo:52-532), without the prefix tree.  Beside the pages
// the manager hands out state slots: one index per live request into arrays
// of per-request state of fixed size.
//
// Plain C++17, no CUDA: the tables are copied to the device by the caller.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <vector>

namespace {

constexpr int ERR_CAPACITY = -1;      // no page or slot left
constexpr int ERR_ARGUMENT = -2;      // bad handle, slot or group
constexpr int ERR_STATE = -3;         // double free, unknown request

struct Group {
  int page_size = 0;
  int num_pages = 0;
  int window = 0;  // 0: every key is kept
  std::vector<int32_t> refcount;
  std::vector<int32_t> free_stack;  // back() is handed out next
  int64_t allocs = 0, frees = 0;
};

struct Request {
  bool live = false;
  int64_t id = 0;
  int reserved_len = 0;   // tokens that pages have been reserved for
  int computed_len = 0;   // tokens whose entries have been written
  // per group: page id per block index, -1 where the window has passed
  std::vector<std::vector<int32_t>> table;
  std::vector<int> first_block;  // per group: blocks below this were given back
};

struct Manager {
  std::vector<Group> groups;
  std::vector<Request> requests;  // index = state slot
  int max_blocks = 0;
};

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

int alloc_page(Group& g) {
  if (g.free_stack.empty()) return ERR_CAPACITY;
  int p = g.free_stack.back();
  g.free_stack.pop_back();
  g.refcount[p] = 1;
  g.allocs++;
  return p;
}

int release_page(Group& g, int p) {
  if (p < 0 || p >= g.num_pages || g.refcount[p] <= 0) return ERR_STATE;
  if (--g.refcount[p] == 0) {
    g.free_stack.push_back(p);
    g.frees++;
    return 1;
  }
  return 0;
}

// Blocks of a request that are wholly below the oldest key the next query
// (at position `len`) can see in a window of `window` keys.
inline int blocks_passed(const Group& g, int len) {
  if (g.window <= 0) return 0;
  int oldest_needed = len - g.window + 1;
  if (oldest_needed <= 0) return 0;
  return oldest_needed / g.page_size;
}

}  // namespace

extern "C" {

void* cm_create(int n_groups, const int* page_size, const int* num_pages, const int* window,
                int max_requests, int max_blocks_per_request) {
  if (n_groups < 0 || max_requests <= 0 || max_blocks_per_request <= 0) return nullptr;  // no group: state slots only
  auto* m = new Manager();
  m->groups.resize(n_groups);
  for (int i = 0; i < n_groups; ++i) {
    Group& g = m->groups[i];
    if (page_size[i] <= 0 || num_pages[i] <= 0 || window[i] < 0) {
      delete m;
      return nullptr;
    }
    g.page_size = page_size[i];
    g.num_pages = num_pages[i];
    g.window = window[i];
    g.refcount.assign(g.num_pages, 0);
    g.free_stack.resize(g.num_pages);
    for (int p = 0; p < g.num_pages; ++p) g.free_stack[p] = g.num_pages - 1 - p;
  }
  m->requests.resize(max_requests);
  m->max_blocks = max_blocks_per_request;
  for (auto& r : m->requests) {
    r.table.assign(n_groups, std::vector<int32_t>());
    r.first_block.assign(n_groups, 0);
    for (auto& t : r.table) t.reserve(max_blocks_per_request);
  }
  return m;
}

void cm_destroy(void* h) { delete static_cast<Manager*>(h); }

// Admit a request: the lowest free state slot, with empty block tables.
int cm_admit(void* h, int64_t id) {
  auto* m = static_cast<Manager*>(h);
  if (!m) return ERR_ARGUMENT;
  for (auto& r : m->requests)
    if (r.live && r.id == id) return ERR_STATE;
  for (size_t s = 0; s < m->requests.size(); ++s) {
    Request& r = m->requests[s];
    if (!r.live) {
      r.live = true;
      r.id = id;
      r.reserved_len = r.computed_len = 0;
      for (size_t g = 0; g < m->groups.size(); ++g) {
        r.table[g].clear();
        r.first_block[g] = 0;
      }
      return static_cast<int>(s);
    }
  }
  return ERR_CAPACITY;
}

int cm_find(void* h, int64_t id) {
  auto* m = static_cast<Manager*>(h);
  if (!m) return ERR_ARGUMENT;
  for (size_t s = 0; s < m->requests.size(); ++s)
    if (m->requests[s].live && m->requests[s].id == id) return static_cast<int>(s);
  return ERR_STATE;
}

// New pages that growing slot `s` to `new_len` tokens takes, per group.
int cm_pages_needed(void* h, int s, int new_len, int* out) {
  auto* m = static_cast<Manager*>(h);
  if (!m || s < 0 || s >= (int)m->requests.size() || !m->requests[s].live) return ERR_ARGUMENT;
  const Request& r = m->requests[s];
  for (size_t g = 0; g < m->groups.size(); ++g) {
    int want = ceil_div(new_len, m->groups[g].page_size);
    int have = static_cast<int>(r.table[g].size());
    out[g] = want > have ? want - have : 0;
  }
  return 0;
}

// Reserve pages so that slot `s` can hold `new_len` tokens: all groups or none.
int cm_reserve(void* h, int s, int new_len) {
  auto* m = static_cast<Manager*>(h);
  if (!m || s < 0 || s >= (int)m->requests.size() || !m->requests[s].live) return ERR_ARGUMENT;
  Request& r = m->requests[s];
  if (new_len < r.reserved_len) return ERR_ARGUMENT;
  for (size_t g = 0; g < m->groups.size(); ++g) {
    Group& grp = m->groups[g];
    int want = ceil_div(new_len, grp.page_size);
    if (want > m->max_blocks) return ERR_CAPACITY;
    int have = static_cast<int>(r.table[g].size());
    if (want - have > (int)grp.free_stack.size()) return ERR_CAPACITY;
  }
  for (size_t g = 0; g < m->groups.size(); ++g) {
    Group& grp = m->groups[g];
    int want = ceil_div(new_len, grp.page_size);
    while ((int)r.table[g].size() < want) r.table[g].push_back(alloc_page(grp));
  }
  r.reserved_len = new_len;
  return 0;
}

// The entries up to `new_len` have been written: give back the pages that a
// group's window has passed.  Returns the number of pages freed.
int cm_advance(void* h, int s, int new_len) {
  auto* m = static_cast<Manager*>(h);
  if (!m || s < 0 || s >= (int)m->requests.size() || !m->requests[s].live) return ERR_ARGUMENT;
  Request& r = m->requests[s];
  if (new_len > r.reserved_len || new_len < r.computed_len) return ERR_ARGUMENT;
  r.computed_len = new_len;
  int freed = 0;
  for (size_t g = 0; g < m->groups.size(); ++g) {
    Group& grp = m->groups[g];
    int passed = blocks_passed(grp, new_len);
    if (passed > (int)r.table[g].size()) passed = (int)r.table[g].size();
    for (int b = r.first_block[g]; b < passed; ++b) {
      if (r.table[g][b] >= 0) {
        if (release_page(grp, r.table[g][b]) < 0) return ERR_STATE;
        r.table[g][b] = -1;
        freed++;
      }
    }
    if (passed > r.first_block[g]) r.first_block[g] = passed;
  }
  return freed;
}

// Give back everything slot `s` holds, and the slot itself.
int cm_release(void* h, int s) {
  auto* m = static_cast<Manager*>(h);
  if (!m || s < 0 || s >= (int)m->requests.size()) return ERR_ARGUMENT;
  Request& r = m->requests[s];
  if (!r.live) return ERR_STATE;
  int freed = 0;
  for (size_t g = 0; g < m->groups.size(); ++g) {
    for (int32_t p : r.table[g]) {
      if (p < 0) continue;
      int rc = release_page(m->groups[g], p);
      if (rc < 0) return ERR_STATE;
      freed += rc;
    }
    r.table[g].clear();
    r.first_block[g] = 0;
  }
  r.live = false;
  r.reserved_len = r.computed_len = 0;
  return freed;
}

// Share the first `n_tokens` (a multiple of every group's page size, inside the
// source's computed length) of slot `src` with the empty slot `dst`: the pages
// are retained, not copied.
int cm_share_prefix(void* h, int src, int dst, int n_tokens) {
  auto* m = static_cast<Manager*>(h);
  if (!m || src < 0 || dst < 0 || src >= (int)m->requests.size() || dst >= (int)m->requests.size()) return ERR_ARGUMENT;
  Request& a = m->requests[src];
  Request& b = m->requests[dst];
  if (!a.live || !b.live || b.reserved_len != 0 || n_tokens > a.computed_len) return ERR_ARGUMENT;
  for (size_t g = 0; g < m->groups.size(); ++g) {
    if (n_tokens % m->groups[g].page_size != 0) return ERR_ARGUMENT;
    int nb = n_tokens / m->groups[g].page_size;
    for (int i = 0; i < nb; ++i)
      if (a.table[g][i] < 0) return ERR_ARGUMENT;
  }
  for (size_t g = 0; g < m->groups.size(); ++g) {
    int nb = n_tokens / m->groups[g].page_size;
    for (int i = 0; i < nb; ++i) {
      m->groups[g].refcount[a.table[g][i]]++;
      b.table[g].push_back(a.table[g][i]);
    }
  }
  b.reserved_len = b.computed_len = n_tokens;
  return 0;
}

// Copy slot `s`'s block table of group `g` into out[0..max); returns its length.
int cm_block_table(void* h, int s, int g, int32_t* out, int max) {
  auto* m = static_cast<Manager*>(h);
  if (!m || s < 0 || s >= (int)m->requests.size() || g < 0 || g >= (int)m->groups.size()) return ERR_ARGUMENT;
  const Request& r = m->requests[s];
  if (!r.live) return ERR_STATE;
  int n = static_cast<int>(r.table[g].size());
  if (n > max) return ERR_CAPACITY;
  if (n) std::memcpy(out, r.table[g].data(), sizeof(int32_t) * n);
  return n;
}

// Plan one step in a single call: for every entry (state slot, token count)
// reserve pages for its new tokens and fill the step's metadata arrays.
//   slots[n], counts[n]   the entries, in batch order
//   want_counts[n], wants the wanted places of each entry (relative to its tokens)
//   meta                  the int32 metadata buffer; off[] gives the word offset of
//                         token-independent fields in this order: positions,
//                         seq_of_token, q_start, kv_len, state_slots, logit_rows,
//                         then per group slot_map, block_table
//   max_blocks            row length of the block tables in meta
//   info out              max tokens of an entry, max keys of an entry, total tokens
// Token ids are copied by the caller.  All or nothing: every entry is checked
// (slot live and named once, places inside its tokens) and the pages that all
// entries need together are counted against each group's free pages before
// anything is reserved or written, so a step that is refused (ERR_CAPACITY when
// the pages do not suffice, ERR_ARGUMENT for a bad slot or place) leaves the
// manager and `meta` as they were.  A reservation left by a step that was
// planned but never committed is given back first.
int cm_plan_step(void* h, int n, const int* slots, const int* counts, const int* want_counts, const int* wants, int32_t* meta,
                 const int* off, int max_blocks, int* info) {
  auto* m = static_cast<Manager*>(h);
  if (!m || n <= 0) return ERR_ARGUMENT;
  const int G = (int)m->groups.size();
  int32_t* positions = meta + off[0];
  int32_t* seq_of = meta + off[1];
  int32_t* q_start = meta + off[2];
  int32_t* kv_len = meta + off[3];
  int32_t* state_slots = meta + off[4];
  int32_t* logit_rows = meta + off[5];
  int row = 0, out = 0, want_at = 0, max_q = 0, max_kv = 0;
  // first pass: nothing is changed until every entry is known to fit
  {
    std::vector<int> need(G, 0);
    std::vector<char> named(m->requests.size(), 0);
    int at = 0;
    for (int i = 0; i < n; ++i) {
      const int s = slots[i], cnt = counts[i];
      if (s < 0 || s >= (int)m->requests.size() || !m->requests[s].live || cnt <= 0 || named[s]) return ERR_ARGUMENT;
      named[s] = 1;
      if (want_counts[i] < 0) return ERR_ARGUMENT;
      for (int w = 0; w < want_counts[i]; ++w) {
        const int place = wants[at++];
        if (place < 0 || place >= cnt) return ERR_ARGUMENT;
      }
      const Request& r = m->requests[s];
      for (int g = 0; g < G; ++g) {
        const int want = ceil_div(r.computed_len + cnt, m->groups[g].page_size);
        if (want > m->max_blocks || want > max_blocks) return ERR_CAPACITY;
        // pages held beyond the computed length come from a step that was planned and not committed
        const int have = std::min((int)r.table[g].size(), ceil_div(r.computed_len, m->groups[g].page_size));
        need[g] += want > have ? want - have : 0;
      }
    }
    for (int g = 0; g < G; ++g) {
      int stale = 0;  // pages that the second pass gives back before it reserves
      for (int i = 0; i < n; ++i) {
        const Request& r = m->requests[slots[i]];
        const int keep = ceil_div(r.computed_len, m->groups[g].page_size);
        if ((int)r.table[g].size() > keep) stale += (int)r.table[g].size() - keep;
      }
      if (need[g] > (int)m->groups[g].free_stack.size() + stale) return ERR_CAPACITY;
    }
  }
  for (int i = 0; i < n; ++i) {
    const int s = slots[i], cnt = counts[i];
    Request& r = m->requests[s];
    const int start = r.computed_len;
    if (r.reserved_len > start) {  // an uncommitted reservation: back to what is written
      for (int g = 0; g < G; ++g) {
        const int keep = ceil_div(start, m->groups[g].page_size);
        while ((int)r.table[g].size() > keep) {
          if (r.table[g].back() >= 0 && release_page(m->groups[g], r.table[g].back()) < 0) return ERR_STATE;
          r.table[g].pop_back();
        }
      }
      r.reserved_len = start;
    }
    int rc = cm_reserve(h, s, start + cnt);
    if (rc != 0) return rc;  // cannot happen after the first pass
    q_start[i] = row;
    kv_len[i] = start + cnt;
    state_slots[i] = s;
    for (int t = 0; t < cnt; ++t) {
      positions[row + t] = start + t;
      seq_of[row + t] = i;
    }
    for (int w = 0; w < want_counts[i]; ++w) {
      const int place = wants[want_at++];
      if (place < 0 || place >= cnt) return ERR_ARGUMENT;
      logit_rows[out++] = row + place;
    }
    for (int g = 0; g < G; ++g) {
      const Group& grp = m->groups[g];
      int32_t* slot_map = meta + off[6 + 2 * g];
      int32_t* table = meta + off[7 + 2 * g] + (size_t)i * max_blocks;
      const int nb = (int)r.table[g].size();
      if (nb > max_blocks) return ERR_CAPACITY;
      for (int b = 0; b < nb; ++b) table[b] = r.table[g][b];
      for (int b = nb; b < max_blocks; ++b) table[b] = -1;
      for (int t = 0; t < cnt; ++t) {
        const int p = start + t;
        slot_map[row + t] = r.table[g][p / grp.page_size] * grp.page_size + p % grp.page_size;
      }
    }
    row += cnt;
    if (cnt > max_q) max_q = cnt;
    if (start + cnt > max_kv) max_kv = start + cnt;
  }
  q_start[n] = row;
  info[0] = max_q;
  info[1] = max_kv;
  info[2] = row;
  return 0;
}

// Advance every entry of a planned step by its token count.
int cm_commit_step(void* h, int n, const int* slots, const int* counts) {
  auto* m = static_cast<Manager*>(h);
  if (!m) return ERR_ARGUMENT;
  for (int i = 0; i < n; ++i) {
    const int s = slots[i];
    if (s < 0 || s >= (int)m->requests.size() || !m->requests[s].live) return ERR_ARGUMENT;
    int rc = cm_advance(h, s, m->requests[s].computed_len + counts[i]);
    if (rc < 0) return rc;
  }
  return 0;
}

int cm_free_pages(void* h, int g) {
  auto* m = static_cast<Manager*>(h);
  if (!m || g < 0 || g >= (int)m->groups.size()) return ERR_ARGUMENT;
  return static_cast<int>(m->groups[g].free_stack.size());
}

int cm_num_pages(void* h, int g) {
  auto* m = static_cast<Manager*>(h);
  if (!m || g < 0 || g >= (int)m->groups.size()) return ERR_ARGUMENT;
  return m->groups[g].num_pages;
}

int cm_reserved_len(void* h, int s) {
  auto* m = static_cast<Manager*>(h);
  if (!m || s < 0 || s >= (int)m->requests.size() || !m->requests[s].live) return ERR_ARGUMENT;
  return m->requests[s].reserved_len;
}

int cm_computed_len(void* h, int s) {
  auto* m = static_cast<Manager*>(h);
  if (!m || s < 0 || s >= (int)m->requests.size() || !m->requests[s].live) return ERR_ARGUMENT;
  return m->requests[s].computed_len;
}

int cm_live_requests(void* h) {
  auto* m = static_cast<Manager*>(h);
  if (!m) return ERR_ARGUMENT;
  int n = 0;
  for (auto& r : m->requests) n += r.live ? 1 : 0;
  return n;
}

int64_t cm_counter(void* h, int g, int which) {
  auto* m = static_cast<Manager*>(h);
  if (!m || g < 0 || g >= (int)m->groups.size()) return ERR_ARGUMENT;
  return which == 0 ? m->groups[g].allocs : m->groups[g].frees;
}

// Recompute every reference count from the tables and compare with the books:
// the number of disagreements (0 when sound).  Checks, per group, that a
// page's count equals the number of table entries naming it, that the free
// stack holds exactly the pages with count 0, each once, and that no table
// is longer than its reservation needs.
int cm_defects(void* h) {
  auto* m = static_cast<Manager*>(h);
  if (!m) return ERR_ARGUMENT;
  int defects = 0;
  for (size_t g = 0; g < m->groups.size(); ++g) {
    const Group& grp = m->groups[g];
    std::vector<int> holders(grp.num_pages, 0), in_free(grp.num_pages, 0);
    for (const auto& r : m->requests) {
      if (!r.live) {
        if (!r.table[g].empty()) defects++;
        continue;
      }
      if ((int)r.table[g].size() != ceil_div(r.reserved_len, grp.page_size)) defects++;
      for (size_t b = 0; b < r.table[g].size(); ++b) {
        int32_t p = r.table[g][b];
        if (p < 0) {
          if ((int)b >= r.first_block[g]) defects++;
          continue;
        }
        if (p >= grp.num_pages) {
          defects++;
          continue;
        }
        holders[p]++;
      }
    }
    for (int32_t p : grp.free_stack) {
      if (p < 0 || p >= grp.num_pages) {
        defects++;
        continue;
      }
      in_free[p]++;
    }
    for (int p = 0; p < grp.num_pages; ++p) {
      if (holders[p] != grp.refcount[p]) defects++;
      if ((grp.refcount[p] == 0) != (in_free[p] == 1)) defects++;
      if (in_free[p] > 1) defects++;
    }
  }
  return defects;
}

// Rolling hash of the whole state, free-stack order included, so two runs can
// be compared (runtime/kv/pool.mojo digest; engine/scheduler.mojo:463-479).
int64_t cm_digest(void* h) {
  auto* m = static_cast<Manager*>(h);
  if (!m) return ERR_ARGUMENT;
  const int64_t MOD = 2147483647, MUL = 1000003;
  int64_t d = 0;
  auto mix = [&](int64_t v) { d = (d * MUL + ((v % MOD) + MOD) % MOD) % MOD; };
  for (const auto& grp : m->groups) {
    for (int32_t rc : grp.refcount) mix(rc);
    for (int32_t p : grp.free_stack) mix(p);
  }
  for (const auto& r : m->requests) {
    mix(r.live);
    if (!r.live) continue;
    mix(r.id);
    mix(r.reserved_len);
    mix(r.computed_len);
    for (const auto& t : r.table)
      for (int32_t p : t) mix(p + 1);
  }
  return d;
}

}  // extern "C"
