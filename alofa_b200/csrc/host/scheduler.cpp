// The scheduler: who runs this tick, as a pure function of its state and of
// what happened since the last tick.  No I/O, no clock, no allocation in step.
//
// It follows the form and the tick order of the reference's scheduler
// (src/alofa/engine/scheduler.mojo:639-767): cancels, engine-reported
// completions, wait-tick increment, arrivals, promotion, decode (one token per
// running request, preempting the newest running request when pages run out),
// starved prefill, first-come prefill (one portion per request per tick under
// one token budget), watermark preemption.  Differences, on purpose:
//   * one book of pages: the free-page count of every cache group comes in
//     with each tick from the cache manager; the scheduler only tracks what
//     its own decisions of this tick take and give back;
//   * sizes are run-time values;
//   * tokens are counted in one place: `n_out` is the number of tokens a
//     request has produced, the first of them by the step that ends its
//     prompt (the reference counts decode ticks and is one short,
//     scheduler.mojo:539-557);
//   * an arrival that does not fit now is deferred, not refused, and "newest"
//     means latest admitted, not highest slot.
#include <cstdint>
#include <cstring>
#include <vector>

namespace {

constexpr int ST_FREE = 0, ST_WAITING = 1, ST_RUNNING = 2;
constexpr int ERR_ARGUMENT = -2, ERR_POOL_TOO_SMALL = -4, ERR_OVERFLOW = -5;
constexpr int ADMIT_COMMITTED = 0, ADMIT_OPTIMISTIC = 1;
constexpr int64_t DIGEST_MOD = 2147483647, DIGEST_MUL = 1000003;

struct Slot {
  int64_t id = 0;
  int prompt_len = 0, max_new = 0, done = 0, n_out = 0, state = ST_FREE, wait_ticks = 0, preempt_count = 0;
  int64_t seq = 0;  // admission order
  bool progressed = false;
  int cache_len() const { return done + (n_out > 0 ? n_out - 1 : 0); }
};

struct Sched {
  int token_budget, max_chunk, max_batch, max_tokens, watermark_permille, max_wait_ticks, admission;
  std::vector<int> page_size, window, capacity;
  std::vector<Slot> slots;
  std::vector<int> free_local, order;
  int64_t tick_seq = 0, preempt_total = 0, next_seq = 1;
};

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Pages a sequence of `len` cached tokens holds in group g (pages a window has
// passed were given back by the cache manager).
int held(const Sched& s, int g, int len) {
  if (len <= 0) return 0;
  int blocks = ceil_div(len, s.page_size[g]);
  if (s.window[g] > 0) {
    int oldest = len - s.window[g] + 1;
    if (oldest > 0) blocks -= oldest / s.page_size[g];
  }
  return blocks;
}

// Most pages a request of `total` tokens ever holds in group g while it is
// prefilled in portions of at most max_chunk tokens.
int worst(const Sched& s, int g, int total) {
  if (s.window[g] <= 0) return ceil_div(total, s.page_size[g]);
  int span = s.window[g] + s.max_chunk;
  if (span > total) span = total;
  return ceil_div(span, s.page_size[g]) + 1;
}

int threshold(const Sched& s, int g) { return (int)((int64_t)s.capacity[g] * s.watermark_permille / 1000); }

int find(const Sched& s, int64_t id) {
  for (size_t i = 0; i < s.slots.size(); ++i)
    if (s.slots[i].state != ST_FREE && s.slots[i].id == id) return (int)i;
  return -1;
}

void clear(Slot& sl) { sl = Slot(); }

struct Out {
  int64_t *p_id, *d_id, *x_id, *f_id;
  int *p_start, *p_end;
  int n_prefill = 0, n_decode = 0, n_preempt = 0, n_finished = 0;
};

// Preempt the newest request that holds pages (latest admitted first); not
// `protect`.  The reference only preempts running requests
// (scheduler.mojo:569-594) so that a tight watermark cannot keep a prompt from
// ever completing; here a prompt portion is only scheduled while it fits
// under the watermark (try_prefill), and the oldest holder is never the victim
// of a newer one, so the oldest live request always finishes.
bool preempt_one(Sched& s, Out& out, int protect) {
  int victim = -1;
  for (size_t i = 0; i < s.slots.size(); ++i) {
    const Slot& sl = s.slots[i];
    if ((int)i == protect || sl.state == ST_FREE || sl.cache_len() <= 0) continue;
    if (victim < 0 || sl.seq > s.slots[victim].seq) victim = (int)i;
  }
  if (victim < 0) return false;
  Slot& v = s.slots[victim];
  // Work of this tick for the victim is withdrawn.  What comes back is what
  // the cache manager holds for it now, plus the pages this tick had set aside
  // for the withdrawn tokens.
  const int len = v.cache_len();
  int before = len;  // tokens the cache manager holds for the victim right now
  for (int i = 0; i < out.n_decode; ++i) {
    if (out.d_id[i] == v.id) {
      for (int j = i + 1; j < out.n_decode; ++j) out.d_id[j - 1] = out.d_id[j];
      out.n_decode--;
      before = len - 1;
      break;
    }
  }
  for (int i = 0; i < out.n_prefill; ++i) {
    if (out.p_id[i] == v.id) {
      before = out.p_start[i];
      for (int j = i + 1; j < out.n_prefill; ++j) {
        out.p_id[j - 1] = out.p_id[j];
        out.p_start[j - 1] = out.p_start[j];
        out.p_end[j - 1] = out.p_end[j];
      }
      out.n_prefill--;
      break;
    }
  }
  for (size_t g = 0; g < s.page_size.size(); ++g)
    s.free_local[g] += held(s, (int)g, before) + ceil_div(len, s.page_size[g]) - ceil_div(before, s.page_size[g]);
  out.x_id[out.n_preempt++] = v.id;
  v.done = 0;
  v.n_out = 0;
  v.wait_ticks = 0;
  v.preempt_count++;
  v.state = ST_WAITING;
  v.progressed = true;  // not prefilled again on the tick that dropped it
  s.preempt_total++;
  return true;
}

int try_prefill(Sched& s, Out& out, int i, int budget) {
  Slot& sl = s.slots[i];
  if (budget <= 0 || sl.state != ST_WAITING || sl.progressed) return budget;
  int remaining = sl.prompt_len - sl.done;
  if (remaining <= 0) return budget;
  int chunk = s.max_chunk < remaining ? s.max_chunk : remaining;
  if (budget < chunk) chunk = budget;
  if (chunk <= 0) return budget;
  const int G = (int)s.page_size.size();
  for (int g = 0; g < G; ++g) {
    int need = ceil_div(sl.done + chunk, s.page_size[g]) - ceil_div(sl.done, s.page_size[g]);
    // left for a later tick when it does not fit under the watermark
    if (s.capacity[g] - s.free_local[g] + need > threshold(s, g)) return budget;
  }
  for (int g = 0; g < G; ++g)
    s.free_local[g] -= ceil_div(sl.done + chunk, s.page_size[g]) - ceil_div(sl.done, s.page_size[g]);
  out.p_id[out.n_prefill] = sl.id;
  out.p_start[out.n_prefill] = sl.done;
  out.p_end[out.n_prefill] = sl.done + chunk;
  out.n_prefill++;
  sl.done += chunk;
  sl.progressed = true;
  sl.wait_ticks = 0;
  if (sl.done >= sl.prompt_len) {
    sl.n_out = 1;  // the step that ends the prompt yields the first token
    if (sl.n_out >= sl.max_new) {
      out.f_id[out.n_finished++] = sl.id;
      clear(sl);
    }
  }
  return budget - chunk;
}

int64_t digest(const Sched& s) {
  int64_t h = 0;
  auto mix = [&](int64_t v) { h = (h * DIGEST_MUL + ((v % DIGEST_MOD) + DIGEST_MOD) % DIGEST_MOD) % DIGEST_MOD; };
  for (const Slot& sl : s.slots) {
    mix(sl.state);
    mix(sl.id);
    mix(sl.prompt_len);
    mix(sl.done);
    mix(sl.n_out);
    mix(sl.max_new);
    mix(sl.wait_ticks);
    mix(sl.preempt_count);
  }
  mix(s.preempt_total);
  return h;
}

}  // namespace

extern "C" {

// cfg: token_budget, max_chunk, max_batch, max_tokens, watermark_permille,
//      max_wait_ticks, admission, n_groups, then per group page_size, window,
//      capacity.  n_groups may be 0 (a model whose layers keep fixed-size state
//      only): no page is ever booked, nothing is ever preempted, and admission is
//      bounded by the request slots alone.
void* sched_create(const int* cfg, int n) {
  if (n < 8) return nullptr;
  auto* s = new Sched();
  s->token_budget = cfg[0];
  s->max_chunk = cfg[1];
  s->max_batch = cfg[2];
  s->max_tokens = cfg[3];
  s->watermark_permille = cfg[4];
  s->max_wait_ticks = cfg[5];
  s->admission = cfg[6];
  int G = cfg[7];
  bool ok = s->token_budget >= 0 && s->max_chunk > 0 && s->max_batch > 0 && s->max_tokens > 0 &&
            s->watermark_permille >= 0 && s->watermark_permille <= 1000 && s->max_wait_ticks >= 0 &&
            (s->admission == ADMIT_COMMITTED || s->admission == ADMIT_OPTIMISTIC) && G >= 0 && n == 8 + 3 * G;
  for (int g = 0; ok && g < G; ++g) {
    s->page_size.push_back(cfg[8 + 3 * g]);
    s->window.push_back(cfg[9 + 3 * g]);
    s->capacity.push_back(cfg[10 + 3 * g]);
    ok = s->page_size[g] > 0 && s->window[g] >= 0 && s->capacity[g] > 0;
  }
  if (!ok) {
    delete s;
    return nullptr;
  }
  s->slots.resize(s->max_batch);
  s->free_local.resize(G);
  s->order.resize(s->max_batch);
  return s;
}

void sched_destroy(void* h) { delete static_cast<Sched*>(h); }

// Would a request of these sizes ever fit, alone?  0 yes; else the reason.
int sched_can_ever_fit(void* h, int prompt_len, int max_new) {
  auto* s = static_cast<Sched*>(h);
  if (!s || prompt_len <= 0 || max_new <= 0) return ERR_ARGUMENT;
  if (prompt_len + max_new > s->max_tokens) return ERR_OVERFLOW;
  for (size_t g = 0; g < s->page_size.size(); ++g)
    if (worst(*s, (int)g, prompt_len + max_new) > threshold(*s, (int)g)) return ERR_POOL_TOO_SMALL;
  return 0;
}

// arr_status out: 1 admitted, 0 deferred (offer it again), 2 blocked by a
// cancel of the same tick, negative: refused for good (the reason).
// info out: tick_seq, preempt_total, digest.
int sched_step(void* h, const int64_t* arr_id, const int* arr_prompt, const int* arr_max_new, int n_arr,
               const int64_t* cancels, int n_cancel, const int64_t* finished, int n_fin, const int* free_pages,
               int* arr_status, int64_t* p_id, int* p_start, int* p_end, int64_t* d_id, int64_t* x_id, int64_t* f_id,
               int* counts, int64_t* info) {
  auto* sp = static_cast<Sched*>(h);
  if (!sp) return ERR_ARGUMENT;
  Sched& s = *sp;
  const int G = (int)s.page_size.size();
  Out out{p_id, d_id, x_id, f_id, p_start, p_end};
  s.tick_seq++;
  for (Slot& sl : s.slots) sl.progressed = false;
  for (int g = 0; g < G; ++g) s.free_local[g] = free_pages[g];

  // 1. cancels: the request leaves at once (its pages were given back by the caller)
  for (int i = 0; i < n_cancel; ++i) {
    int at = find(s, cancels[i]);
    if (at >= 0) clear(s.slots[at]);
  }
  // 2. completions the engine saw (end-of-sequence token, stop id)
  for (int i = 0; i < n_fin; ++i) {
    int at = find(s, finished[i]);
    if (at >= 0) clear(s.slots[at]);
  }
  // 3. the waiting counters of requests already queued go up by one; this tick's arrivals are queued after this, with a count of 0
  for (Slot& sl : s.slots)
    if (sl.state == ST_WAITING) sl.wait_ticks++;

  // 4. arrivals, first come first admitted; a deferred arrival defers all behind it
  bool deferring = false;
  for (int i = 0; i < n_arr; ++i) {
    bool blocked = false;
    for (int j = 0; j < n_cancel; ++j) blocked |= cancels[j] == arr_id[i];
    if (blocked) {
      arr_status[i] = 2;
      continue;
    }
    if (arr_prompt[i] <= 0 || arr_max_new[i] <= 0 || find(s, arr_id[i]) >= 0) {
      arr_status[i] = ERR_ARGUMENT;
      continue;
    }
    int fit = sched_can_ever_fit(h, arr_prompt[i], arr_max_new[i]);
    if (fit != 0) {
      arr_status[i] = fit;
      continue;
    }
    if (deferring) {
      arr_status[i] = 0;
      continue;
    }
    int slot = -1;
    for (size_t k = 0; k < s.slots.size() && slot < 0; ++k)
      if (s.slots[k].state == ST_FREE) slot = (int)k;
    bool fits = slot >= 0;
    for (int g = 0; fits && g < G; ++g) {
      int64_t load = 0;
      if (s.admission == ADMIT_COMMITTED) {
        // everything live may grow to its full length: no preemption can follow
        for (const Slot& sl : s.slots)
          if (sl.state != ST_FREE) load += worst(s, g, sl.prompt_len + sl.max_new);
        load += worst(s, g, arr_prompt[i] + arr_max_new[i]);
      } else {
        // what is held now, what waiting prompts still owe, and this prompt
        load = s.capacity[g] - s.free_local[g];
        for (const Slot& sl : s.slots)
          if (sl.state == ST_WAITING) load += worst(s, g, sl.prompt_len) - held(s, g, sl.done);
        load += worst(s, g, arr_prompt[i] + 1);
      }
      fits = load <= threshold(s, g);
    }
    if (!fits) {
      arr_status[i] = 0;
      deferring = true;
      continue;
    }
    Slot& sl = s.slots[slot];
    clear(sl);
    sl.id = arr_id[i];
    sl.prompt_len = arr_prompt[i];
    sl.max_new = arr_max_new[i];
    sl.state = ST_WAITING;
    sl.seq = s.next_seq++;
    arr_status[i] = 1;
  }

  // 5. promotion: a request whose prompt is done decodes from now on
  for (Slot& sl : s.slots)
    if (sl.state == ST_WAITING && sl.prompt_len > 0 && sl.done >= sl.prompt_len) {
      sl.state = ST_RUNNING;
      sl.wait_ticks = 0;
    }

  int budget = s.token_budget;
  // 6. the token budget is spent on decoding first: every running request gets one token, walked in slot order
  for (size_t i = 0; i < s.slots.size() && budget > 0; ++i) {
    Slot& sl = s.slots[i];
    if (sl.state != ST_RUNNING || sl.progressed) continue;
    const int len = sl.cache_len();
    bool room = false;
    while (!room) {
      room = true;
      for (int g = 0; g < G; ++g) {
        int need = ceil_div(len + 1, s.page_size[g]) - ceil_div(len, s.page_size[g]);
        if (need > s.free_local[g]) room = false;
      }
      if (!room && !preempt_one(s, out, (int)i)) {
        counts[0] = out.n_prefill;
        counts[1] = out.n_decode;
        counts[2] = out.n_preempt;
        counts[3] = out.n_finished;
        return ERR_POOL_TOO_SMALL;
      }
    }
    for (int g = 0; g < G; ++g) s.free_local[g] -= ceil_div(len + 1, s.page_size[g]) - ceil_div(len, s.page_size[g]);
    sl.n_out++;
    sl.progressed = true;
    out.d_id[out.n_decode++] = sl.id;
    budget--;
    if (sl.n_out >= sl.max_new) {
      out.f_id[out.n_finished++] = sl.id;
      clear(sl);
    }
  }

  // waiting requests in admission order
  int n_wait = 0;
  for (size_t i = 0; i < s.slots.size(); ++i)
    if (s.slots[i].state == ST_WAITING) s.order[n_wait++] = (int)i;
  for (int a = 1; a < n_wait; ++a) {
    int v = s.order[a], b = a - 1;
    while (b >= 0 && s.slots[s.order[b]].seq > s.slots[v].seq) {
      s.order[b + 1] = s.order[b];
      --b;
    }
    s.order[b + 1] = v;
  }
  // 7. latency guard: who has waited max_wait_ticks goes before other waiting requests
  for (int a = 0; a < n_wait; ++a)
    if (s.slots[s.order[a]].wait_ticks >= s.max_wait_ticks) budget = try_prefill(s, out, s.order[a], budget);
  // 8. first come, first prefilled; one portion per request per tick
  for (int a = 0; a < n_wait; ++a) budget = try_prefill(s, out, s.order[a], budget);

  // 9. watermark: above it, the newest running request is recomputed later
  for (int g = 0; g < G; ++g)
    while (s.capacity[g] - s.free_local[g] > threshold(s, g))
      if (!preempt_one(s, out, -1)) break;

  counts[0] = out.n_prefill;
  counts[1] = out.n_decode;
  counts[2] = out.n_preempt;
  counts[3] = out.n_finished;
  info[0] = s.tick_seq;
  info[1] = s.preempt_total;
  info[2] = digest(s);
  return 0;
}

// counts: live, waiting, running
void sched_counts(void* h, int* out) {
  auto* s = static_cast<Sched*>(h);
  out[0] = out[1] = out[2] = 0;
  if (!s) return;
  for (const Slot& sl : s->slots) {
    out[0] += sl.state != ST_FREE;
    out[1] += sl.state == ST_WAITING;
    out[2] += sl.state == ST_RUNNING;
  }
}

// out: state, prompt_len, max_new, done, n_out, wait_ticks, preempt_count, cache_len; returns 0 or -1
int sched_request(void* h, int64_t id, int* out) {
  auto* s = static_cast<Sched*>(h);
  if (!s) return -1;
  int at = find(*s, id);
  if (at < 0) return -1;
  const Slot& sl = s->slots[at];
  out[0] = sl.state;
  out[1] = sl.prompt_len;
  out[2] = sl.max_new;
  out[3] = sl.done;
  out[4] = sl.n_out;
  out[5] = sl.wait_ticks;
  out[6] = sl.preempt_count;
  out[7] = sl.cache_len();
  return 0;
}

}  // extern "C"
