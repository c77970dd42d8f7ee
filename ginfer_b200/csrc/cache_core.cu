// Host-side bookkeeping of the paged cache in C++ (no device code): page pools with an owner per
// page, request slots, block tables, reservation and commit of a step's tokens, windowed groups
// that give pages back.  The same rules as ginfer_b200/cache/manager.py, which stays as the
// readable statement of them and as the oracle of the tests; this is what the engine runs.
//
// Reference: ginfer/engine/block_manager.{h,cc} (one page id for all layers, a free deque that is
// searched on every allocation, a prompt's pages taken whole at admission).  Here: a LIFO free
// stack and an owner array per layer group (double hand-outs, double returns and foreign returns
// are errors), pages taken step by step, pages of a windowed group returned as soon as no later
// token can see them.
//
// The block tables are int32 arrays [slots][width] that the caller owns (numpy) and this code
// writes; a request is addressed by its slot.
#include <stdint.h>

#include <algorithm>
#include <cstdio>
#include <string>
#include <vector>

#define GF_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

enum Code { OK = 0, OUT_OF_PAGES = 1, POOL_ERROR = 2, NO_FREE_SLOT = 3, BAD_VALUE = 4, NOT_LIVE = 5,
            CHECK_FAILED = 6 };

struct Pool {
  int num_pages = 0;
  std::vector<int> free_;            // back() goes out first
  std::vector<int64_t> owner;        // -1: free
};

struct Req {
  bool live = false;
  int64_t owner = -1;
  int num_tokens = 0, reserved = 0;
  std::vector<int> first_page, next_page;   // per group
};

struct Manager {
  int G = 0, page_size = 0, max_seqs = 0, max_seq_len = 0, width = 0;
  std::vector<int> windows;
  std::vector<Pool> pools;
  std::vector<int32_t*> tables;      // [G] -> [max_seqs][width]
  std::vector<int> free_slots;       // back() goes out first
  std::vector<Req> reqs;             // by slot
  int64_t next_owner = 0;
  std::string error;

  int fail(Code c, const std::string& msg) {
    error = msg;
    return c;
  }
  int32_t* row(int g, int slot) { return tables[g] + (size_t)slot * width; }
  int new_pages(int next_page, int have, int n_new) const {
    const int end_page = (have + n_new + page_size - 1) / page_size;
    return end_page > next_page ? end_page - next_page : 0;
  }
  int give_back(int g, int page, int64_t owner) {
    Pool& p = pools[g];
    char buf[160];
    if (page < 0 || page >= p.num_pages) {
      snprintf(buf, sizeof buf, "page %d is not of this pool", page);
      return fail(POOL_ERROR, buf);
    }
    if (p.owner[page] < 0) {
      snprintf(buf, sizeof buf, "page %d is returned twice", page);
      return fail(POOL_ERROR, buf);
    }
    if (p.owner[page] != owner) {
      snprintf(buf, sizeof buf, "page %d is held by %lld, not by %lld", page,
               (long long)p.owner[page], (long long)owner);
      return fail(POOL_ERROR, buf);
    }
    p.owner[page] = -1;
    p.free_.push_back(page);
    return OK;
  }
};

bool live_slot(Manager* m, int slot) {
  return slot >= 0 && slot < m->max_seqs && m->reqs[slot].live;
}

}  // namespace

GF_EXPORT void* gf_cm_create(int num_groups, const int* pages_per_group, const int* windows,
                             int page_size, int max_num_seqs, int max_seq_len,
                             int32_t* const* tables) {
  if (num_groups <= 0 || page_size <= 0 || max_num_seqs <= 0 || max_seq_len <= 0) return nullptr;
  auto* m = new Manager();
  m->G = num_groups, m->page_size = page_size, m->max_seqs = max_num_seqs;
  m->max_seq_len = max_seq_len;
  m->width = (max_seq_len + page_size - 1) / page_size;
  m->windows.assign(windows, windows + num_groups);
  m->pools.resize(num_groups);
  for (int g = 0; g < num_groups; ++g) {
    Pool& p = m->pools[g];
    if (pages_per_group[g] <= 0) {
      delete m;
      return nullptr;
    }
    p.num_pages = pages_per_group[g];
    p.owner.assign(p.num_pages, -1);
    p.free_.resize(p.num_pages);
    for (int i = 0; i < p.num_pages; ++i) p.free_[i] = p.num_pages - 1 - i;   // page 0 goes out first
    m->tables.push_back(tables[g]);
    std::fill(tables[g], tables[g] + (size_t)max_num_seqs * m->width, -1);
  }
  m->free_slots.resize(max_num_seqs);
  for (int i = 0; i < max_num_seqs; ++i) m->free_slots[i] = max_num_seqs - 1 - i;
  m->reqs.resize(max_num_seqs);
  return m;
}

GF_EXPORT void gf_cm_destroy(void* h) { delete (Manager*)h; }
GF_EXPORT const char* gf_cm_error(void* h) { return ((Manager*)h)->error.c_str(); }
GF_EXPORT int gf_cm_table_width(void* h) { return ((Manager*)h)->width; }
GF_EXPORT int gf_cm_free_slots(void* h) { return (int)((Manager*)h)->free_slots.size(); }

GF_EXPORT void gf_cm_free_pages(void* h, int* out) {
  auto* m = (Manager*)h;
  for (int g = 0; g < m->G; ++g) out[g] = (int)m->pools[g].free_.size();
}

// A slot for a new request (no pages yet); *slot = -1 if none is free.
GF_EXPORT int gf_cm_admit(void* h, int* slot) {
  auto* m = (Manager*)h;
  *slot = -1;
  if (m->free_slots.empty()) {
    char buf[80];
    snprintf(buf, sizeof buf, "all %d request slots are taken", m->max_seqs);
    return m->fail(NO_FREE_SLOT, buf);
  }
  const int s = m->free_slots.back();
  m->free_slots.pop_back();
  Req& r = m->reqs[s];
  r.live = true;
  r.owner = m->next_owner++;
  r.num_tokens = r.reserved = 0;
  r.first_page.assign(m->G, 0);
  r.next_page.assign(m->G, 0);
  *slot = s;
  return OK;
}

// out[0] = num_tokens, out[1] = reserved, out[2] = owner (low 31 bits), then first_page[G],
// next_page[G].
GF_EXPORT int gf_cm_get(void* h, int slot, long long* out) {
  auto* m = (Manager*)h;
  if (!live_slot(m, slot)) return m->fail(NOT_LIVE, "no live request holds this slot");
  const Req& r = m->reqs[slot];
  out[0] = r.num_tokens, out[1] = r.reserved, out[2] = r.owner;
  for (int g = 0; g < m->G; ++g) out[3 + g] = r.first_page[g], out[3 + m->G + g] = r.next_page[g];
  return OK;
}

// Tokens in the cache of each of `count` requests.
GF_EXPORT int gf_cm_lengths(void* h, const int* slots, int count, int* out) {
  auto* m = (Manager*)h;
  for (int i = 0; i < count; ++i) {
    if (!live_slot(m, slots[i])) return m->fail(NOT_LIVE, "no live request holds this slot");
    out[i] = m->reqs[slots[i]].num_tokens;
  }
  return OK;
}

// Pages per group that reserve would take for n_new more tokens; slot < 0: a request not admitted.
GF_EXPORT int gf_cm_pages_needed(void* h, int slot, int n_new, int* out) {
  auto* m = (Manager*)h;
  if (slot < 0) {
    for (int g = 0; g < m->G; ++g) out[g] = (n_new + m->page_size - 1) / m->page_size;
    return OK;
  }
  if (!live_slot(m, slot)) return m->fail(NOT_LIVE, "no live request holds this slot");
  const Req& r = m->reqs[slot];
  for (int g = 0; g < m->G; ++g)
    out[g] = m->new_pages(r.next_page[g], r.num_tokens + r.reserved, n_new);
  return OK;
}

// The pages a whole step needs per group: entries of admitted requests (slot >= 0) and new ones.
GF_EXPORT int gf_cm_step_need(void* h, const int* slots, const int* n_new, int count, int* need,
                              int* over_len) {
  auto* m = (Manager*)h;
  std::fill(need, need + m->G, 0);
  *over_len = -1;
  for (int i = 0; i < count; ++i) {
    int have = 0;
    if (slots[i] >= 0) {
      if (!live_slot(m, slots[i])) return m->fail(NOT_LIVE, "no live request holds this slot");
      const Req& r = m->reqs[slots[i]];
      have = r.num_tokens + r.reserved;
      for (int g = 0; g < m->G; ++g) need[g] += m->new_pages(r.next_page[g], have, n_new[i]);
    } else {
      for (int g = 0; g < m->G; ++g) need[g] += (n_new[i] + m->page_size - 1) / m->page_size;
    }
    if (have + n_new[i] > m->max_seq_len && *over_len < 0) *over_len = i;
  }
  return OK;
}

// Pages for the next n_new tokens of the request, in every group or (if one pool is short) in none.
GF_EXPORT int gf_cm_reserve(void* h, int slot, int n_new) {
  auto* m = (Manager*)h;
  if (!live_slot(m, slot)) return m->fail(NOT_LIVE, "no live request holds this slot");
  Req& r = m->reqs[slot];
  const int have = r.num_tokens + r.reserved;
  char buf[200];
  if (n_new < 0 || have + n_new > m->max_seq_len) {
    snprintf(buf, sizeof buf, "the request would hold %d tokens; max_seq_len is %d", have + n_new,
             m->max_seq_len);
    return m->fail(BAD_VALUE, buf);
  }
  std::vector<int> need(m->G);
  for (int g = 0; g < m->G; ++g) {
    need[g] = m->new_pages(r.next_page[g], have, n_new);
    if (need[g] > (int)m->pools[g].free_.size()) {
      snprintf(buf, sizeof buf, "group %d: the request needs %d pages for %d tokens, %d are free", g,
               need[g], n_new, (int)m->pools[g].free_.size());
      return m->fail(OUT_OF_PAGES, buf);
    }
  }
  for (int g = 0; g < m->G; ++g) {
    Pool& p = m->pools[g];
    int32_t* row = m->row(g, slot);
    for (int k = 0; k < need[g]; ++k) {
      const int page = p.free_.back();
      p.free_.pop_back();
      if (p.owner[page] >= 0) {
        snprintf(buf, sizeof buf, "page %d was on the free list while held by %lld", page,
                 (long long)p.owner[page]);
        return m->fail(POOL_ERROR, buf);
      }
      p.owner[page] = r.owner;
      row[r.next_page[g]++] = page;
    }
  }
  r.reserved += n_new;
  return OK;
}

// n reserved tokens are now in the cache; windowed groups give back the pages no later token sees
// (a page whose last position is <= num_tokens - window is dead).
GF_EXPORT int gf_cm_commit(void* h, int slot, int n) {
  auto* m = (Manager*)h;
  if (!live_slot(m, slot)) return m->fail(NOT_LIVE, "no live request holds this slot");
  Req& r = m->reqs[slot];
  if (n < 0 || n > r.reserved) {
    char buf[120];
    snprintf(buf, sizeof buf, "commit of %d tokens but only %d are reserved", n, r.reserved);
    return m->fail(BAD_VALUE, buf);
  }
  r.reserved -= n;
  r.num_tokens += n;
  for (int g = 0; g < m->G; ++g) {
    const int w = m->windows[g];
    if (w <= 0) continue;
    int dead_end = std::max(0, r.num_tokens - w + 1) / m->page_size;
    dead_end = std::min(dead_end, r.next_page[g]);
    int32_t* row = m->row(g, slot);
    for (int lp = r.first_page[g]; lp < dead_end; ++lp) {
      if (int rc = m->give_back(g, row[lp], r.owner)) return rc;
      row[lp] = -1;
    }
    if (dead_end > r.first_page[g]) r.first_page[g] = dead_end;
  }
  return OK;
}

GF_EXPORT int gf_cm_reserve_many(void* h, const int* slots, const int* n_new, int count) {
  for (int i = 0; i < count; ++i)
    if (int rc = gf_cm_reserve(h, slots[i], n_new[i])) return rc;
  return OK;
}

GF_EXPORT int gf_cm_commit_many(void* h, const int* slots, const int* n, int count) {
  for (int i = 0; i < count; ++i)
    if (int rc = gf_cm_commit(h, slots[i], n[i])) return rc;
  return OK;
}

// Every page of the request goes back; with keep_slot it stays admitted with nothing cached.
GF_EXPORT int gf_cm_release(void* h, int slot, int keep_slot) {
  auto* m = (Manager*)h;
  if (!live_slot(m, slot)) return m->fail(NOT_LIVE, "no live request holds this slot");
  Req& r = m->reqs[slot];
  for (int g = 0; g < m->G; ++g) {
    int32_t* row = m->row(g, slot);
    for (int lp = r.first_page[g]; lp < r.next_page[g]; ++lp)
      if (row[lp] >= 0)
        if (int rc = m->give_back(g, row[lp], r.owner)) return rc;
    std::fill(row, row + r.next_page[g], -1);
    r.first_page[g] = r.next_page[g] = 0;
  }
  r.num_tokens = r.reserved = 0;
  if (!keep_slot) {
    r.live = false;
    m->free_slots.push_back(slot);
  }
  return OK;
}

// No page lost, held twice, or in a table without being held by that request.
GF_EXPORT int gf_cm_check(void* h) {
  auto* m = (Manager*)h;
  char buf[200];
  for (int g = 0; g < m->G; ++g) {
    Pool& p = m->pools[g];
    std::vector<int> state(p.num_pages, 0);          // 1: on the free list, 2: in a live table
    for (int page : p.free_) {
      if (page < 0 || page >= p.num_pages || state[page]) {
        snprintf(buf, sizeof buf, "group %d: page %d is on the free list twice", g, page);
        return m->fail(CHECK_FAILED, buf);
      }
      if (p.owner[page] >= 0) {
        snprintf(buf, sizeof buf, "group %d: page %d is both free and held", g, page);
        return m->fail(CHECK_FAILED, buf);
      }
      state[page] = 1;
    }
    for (int s = 0; s < m->max_seqs; ++s) {
      const Req& r = m->reqs[s];
      const int32_t* row = m->row(g, s);
      if (!r.live) {
        for (int lp = 0; lp < m->width; ++lp)
          if (row[lp] >= 0) {
            snprintf(buf, sizeof buf, "group %d: the free slot %d lists page %d", g, s, row[lp]);
            return m->fail(CHECK_FAILED, buf);
          }
        continue;
      }
      for (int lp = 0; lp < m->width; ++lp) {
        const bool inside = lp >= r.first_page[g] && lp < r.next_page[g];
        if (inside && row[lp] < 0) {
          snprintf(buf, sizeof buf, "group %d: slot %d has a hole at logical page %d", g, s, lp);
          return m->fail(CHECK_FAILED, buf);
        }
        if (!inside && row[lp] >= 0) {
          snprintf(buf, sizeof buf, "group %d: slot %d lists a page it gave back", g, s);
          return m->fail(CHECK_FAILED, buf);
        }
        if (!inside) continue;
        const int page = row[lp];
        if (page >= p.num_pages || state[page]) {
          snprintf(buf, sizeof buf, "group %d: page %d is listed twice (or free and listed)", g,
                   page);
          return m->fail(CHECK_FAILED, buf);
        }
        if (p.owner[page] != r.owner) {
          snprintf(buf, sizeof buf, "group %d: page %d is listed by slot %d but held by another", g,
                   page, s);
          return m->fail(CHECK_FAILED, buf);
        }
        state[page] = 2;
      }
    }
    for (int page = 0; page < p.num_pages; ++page)
      if (!state[page]) {
        snprintf(buf, sizeof buf, "group %d: page %d is lost (neither free nor in a table)", g,
                 page);
        return m->fail(CHECK_FAILED, buf);
      }
  }
  // slots: free once or live once
  std::vector<int> seen(m->max_seqs, 0);
  for (int s : m->free_slots) {
    if (s < 0 || s >= m->max_seqs || seen[s] || m->reqs[s].live)
      return m->fail(CHECK_FAILED, "a slot is free twice or free and live");
    seen[s] = 1;
  }
  for (int s = 0; s < m->max_seqs; ++s)
    if (!seen[s] && !m->reqs[s].live) return m->fail(CHECK_FAILED, "a slot is lost");
  return OK;
}

// ----------------------------------------------------------------------------- one scheduling decision
// The order of work of ginfer_b200/engine/scheduler.py (which stays as the statement of the rules
// and runs when the manager is the Python one): (1) one token for every running request that is
// decoding, oldest first; a request that needs a page takes it from the most recently admitted
// other running request that is not yet in the batch, which is preempted (pages back, slot kept,
// front of the waiting queue, computed again from its first token); (2) portions for running
// requests still in their prompt; (3) admission, oldest first, no overtaking, while a slot, budget
// and pages for a first portion are there; (4) if nothing could move, the youngest running request
// is preempted and the decision is taken again, or a request that is alone is given up.
//
// Requests come as entries 0 .. nr - 1 (running, in order of admission) and nr .. nr + nw - 1
// (waiting, in queue order): slot (-1: none yet), tokens (prompt + output), computed.  The function
// releases and admits through the manager itself.  Results: the batch (entry, start, n, sample),
// the new running and waiting orders, per entry the slot, how often it was preempted and whether
// it was given up (out of pages).
namespace {

struct Sched {
  Manager* m;
  std::vector<int> slot, tokens, computed, preempts, dropped;
  std::vector<int> running, waiting;          // entry indices
  std::vector<int> promised;
  std::vector<int> batch;                     // 4 ints an action
  std::vector<char> in_batch;
  int budget = 0;

  void pages_needed(int e, int n, std::vector<int>& need) const {
    need.resize(m->G);
    if (slot[e] < 0) {
      for (int g = 0; g < m->G; ++g) need[g] = (n + m->page_size - 1) / m->page_size;
      return;
    }
    const Req& r = m->reqs[slot[e]];
    for (int g = 0; g < m->G; ++g)
      need[g] = m->new_pages(r.next_page[g], r.num_tokens + r.reserved, n);
  }
  bool fits(const std::vector<int>& need) const {
    for (int g = 0; g < m->G; ++g)
      if (need[g] > (int)m->pools[g].free_.size() - promised[g]) return false;
    return true;
  }
  bool can_reserve(int e, int n) const {
    std::vector<int> need;
    pages_needed(e, n, need);
    return fits(need);
  }
  int fit(int e, int want) const {
    if (want <= 0) return 0;
    if (can_reserve(e, want)) return want;
    int free_pages = 1 << 30;
    for (int g = 0; g < m->G; ++g)
      free_pages = std::min(free_pages, (int)m->pools[g].free_.size() - promised[g]);
    if (free_pages < 0) return 0;
    int held_end = 0;
    if (slot[e] >= 0) {
      const Req& r = m->reqs[slot[e]];
      held_end = *std::min_element(r.next_page.begin(), r.next_page.end()) * m->page_size;
    }
    const int room = std::max(0, held_end - computed[e]) + free_pages * m->page_size;
    int n = std::min(want, room);
    while (n > 0 && !can_reserve(e, n)) --n;
    return n;
  }
  void promise(int e, int n) {
    std::vector<int> need;
    pages_needed(e, n, need);
    for (int g = 0; g < m->G; ++g) promised[g] += need[g];
  }
  void take(int e, int start, int n, bool sample) {
    batch.push_back(e), batch.push_back(start), batch.push_back(n), batch.push_back(sample);
    in_batch[e] = 1;
    budget -= n;
  }
  int preempt(int e) {
    if (int rc = gf_cm_release(m, slot[e], 1)) return rc;
    computed[e] = 0;
    ++preempts[e];
    running.erase(std::find(running.begin(), running.end(), e));
    waiting.insert(waiting.begin(), e);
    return OK;
  }
  int give_up(int e) {
    dropped[e] = 1;
    auto it = std::find(running.begin(), running.end(), e);
    if (it != running.end()) running.erase(it);
    if (slot[e] >= 0) {
      if (int rc = gf_cm_release(m, slot[e], 0)) return rc;
      slot[e] = -1;
    }
    return OK;
  }
  bool is_running(int e) const {
    return std::find(running.begin(), running.end(), e) != running.end();
  }

  int decide(int max_num_seqs, int full_budget) {
    for (;;) {
      budget = full_budget;
      std::fill(promised.begin(), promised.end(), 0);
      batch.clear();
      std::fill(in_batch.begin(), in_batch.end(), 0);
      bool any_dropped = false;
      // 1. decoding requests, oldest first
      const std::vector<int> snapshot = running;
      std::vector<int> need;
      for (int e : snapshot) {
        if (!is_running(e) || tokens[e] - computed[e] != 1) continue;
        if (budget <= 0) break;
        pages_needed(e, 1, need);
        while (!fits(need)) {
          int victim = -1;
          for (int r : running)
            if (r != e && !in_batch[r]) victim = r;          // the last one: most recently admitted
          if (victim >= 0) {
            if (int rc = preempt(victim)) return rc;
          } else if (running.size() > 1 || !batch.empty()) {
            break;                                           // others hold this step's pages: wait
          } else {
            if (int rc = give_up(e)) return rc;
            any_dropped = true;
            break;
          }
        }
        if (!is_running(e) || !fits(need)) continue;
        for (int g = 0; g < m->G; ++g) promised[g] += need[g];
        take(e, computed[e], 1, true);
      }
      // 2. running requests still feeding their prompt
      const std::vector<int> snapshot2 = running;
      for (int e : snapshot2) {
        const int left = tokens[e] - computed[e];
        if (!is_running(e) || left <= 1 || budget <= 0) continue;
        const int n = fit(e, std::min(left, budget));
        if (n <= 0) continue;
        promise(e, n);
        take(e, computed[e], n, n == left);
      }
      // 3. admission, oldest first, no overtaking
      while (!waiting.empty() && budget > 0 && (int)running.size() < max_num_seqs) {
        const int e = waiting.front();
        if (slot[e] < 0 && m->free_slots.empty()) break;
        const int left = tokens[e];
        const int n = fit(e, std::min(left, budget));
        if (n <= 0) break;
        waiting.erase(waiting.begin());
        if (slot[e] < 0) {
          int s = -1;
          if (int rc = gf_cm_admit(m, &s)) return rc;
          slot[e] = s;
        }
        running.push_back(e);
        promise(e, n);
        take(e, 0, n, n == left);
      }
      // 4. nothing could move although requests are live
      if (batch.empty() && !any_dropped && (!running.empty() || !waiting.empty())) {
        if (running.size() > 1) {
          if (int rc = preempt(running.back())) return rc;
          continue;                                          // decide again
        }
        if (!running.empty()) {
          if (int rc = give_up(running[0])) return rc;
        } else {
          const int e = waiting.front();
          waiting.erase(waiting.begin());
          if (int rc = give_up(e)) return rc;
        }
      }
      return OK;
    }
  }
};

}  // namespace

// in: nr, nw, slot/tokens/computed [nr + nw].  out: slot [nr + nw] (updated in place), preempts
// [nr + nw], dropped [nr + nw], batch [4 * (nr + nw)] with *n_batch actions, order [nr + nw] =
// the new running order then the new waiting order, with *n_running.
GF_EXPORT int gf_sched_decide(void* h, int budget, int max_num_seqs, int nr, int nw, int* slot,
                              const int* tokens, const int* computed, int* preempts, int* dropped,
                              int* batch, int* n_batch, int* order, int* n_running) {
  auto* m = (Manager*)h;
  const int n = nr + nw;
  Sched s;
  s.m = m;
  s.slot.assign(slot, slot + n);
  s.tokens.assign(tokens, tokens + n);
  s.computed.assign(computed, computed + n);
  s.preempts.assign(n, 0);
  s.dropped.assign(n, 0);
  s.in_batch.assign(n, 0);
  s.promised.assign(m->G, 0);
  for (int i = 0; i < nr; ++i) s.running.push_back(i);
  for (int i = nr; i < n; ++i) s.waiting.push_back(i);
  const int rc = s.decide(max_num_seqs, budget);
  if (rc) return rc;
  std::copy(s.slot.begin(), s.slot.end(), slot);
  std::copy(s.preempts.begin(), s.preempts.end(), preempts);
  std::copy(s.dropped.begin(), s.dropped.end(), dropped);
  *n_batch = (int)s.batch.size() / 4;
  std::copy(s.batch.begin(), s.batch.end(), batch);
  *n_running = (int)s.running.size();
  int k = 0;
  for (int e : s.running) order[k++] = e;
  for (int e : s.waiting) order[k++] = e;
  return OK;
}
