// Host-side tree splitter (no device code): the native twin of ft_b200.planner.plan_b200, which stays the
// specification - the tests require both to produce identical tables.  It turns the radix tree into balanced
// (node KV chunk x request tile) tasks for one B200 and emits the nine int32 tables of the reference plan
// format (kernel_bench/fasttree.py:193-262).
//
// Steps: (1) greedy walk over the parent->child edges, breadth first, children in id order, on a cost model in
// streamed-byte equivalents (K/V re-read by a child that carries its parent's KV, fp32 partial rows written and
// read back, a fixed cost per CTA, tensor-core time); (2) request tile = rows_per_cta / G requests; (3) KV chunks
// from a global byte target = streamed bytes of the step / (SMs x CTAs per SM x waves), equal chunks per node on
// 64-token boundaries and never below min_chunk; (4) tasks with more requests than the small tile first (phase
// 0), longest first inside each phase (stable).  All cost arithmetic is IEEE double in the same order as the
// Python code, so the decisions agree bit for bit.
#include <algorithm>
#include <climits>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <deque>
#include <new>
#include <numeric>
#include <queue>
#include <vector>

#include "fasttree_b200.h"

namespace {

struct Model {
  int num_sms = 148, ctas_per_sm = 2;
  double waves = 1.0;
  int tile_tokens = 64, rows_per_cta = 64, min_chunk = 128, nominal_split = 512;
  double ridge_flop_per_byte = 90.0;
  int task_overhead_bytes = 16384, elem_bytes = 2;
  int group_member_tokens = 128, group_min_members = 6;
};

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

double task_cost(int64_t n_req, int64_t length, int group, int head_dim, const Model& m) {
  if (n_req <= 0 || length <= 0) return 0.0;
  const int64_t rows = n_req * group;
  const int64_t row_blocks = ceil_div(rows, m.rows_per_cta);
  const int64_t chunks = ceil_div(length, m.nominal_split);
  const double stream = (double)(row_blocks * length * 2 * head_dim * m.elem_bytes);
  const double tensor = (double)(ceil_div(rows, 16) * 16 * length * 4 * head_dim) / m.ridge_flop_per_byte;
  const double partial = (double)(chunks * rows * (head_dim + 1) * 4 * 2);
  return std::max(stream, tensor) + partial + (double)(row_blocks * chunks * m.task_overhead_bytes);
}

}  // namespace

struct ft_plan {
  std::vector<int32_t> kv_entries, kv_offs, kv_lens, q_entries, q_offs, q_lens, r2v_entries, r2v_offs, r2v_lens;
  std::vector<int32_t> assignments;
  std::vector<int32_t> q_ranges;  // [partial rows][2] when the plan holds groups of short nodes, else empty
  std::vector<int32_t> aux_segments;  // serving plans with groups: per member {source position, length, position in the auxiliary table, room}
  ft_plan_info info;
};

namespace {

// Addressing of the serving path: a node's KV (and that of the ancestors it carries) is ONE run of positions in
// an existing row-id table (SGLang's flattened req_to_token): [base[i] + offset[top carried ancestor],
// base[i] + offset[i] + seqlen[i]).  No row-id table is emitted; vnode_to_kv_offs are positions in that table.
// `extra` pairings (one request each: its private tail) join the byte budget and come last in emission order.
// tail_room >= 0 lets short nodes and tails run as groups (one many-row vnode, per-row token ranges): a group's row
// ids cannot be one run of the table, so they go to an auxiliary table that the caller fills on the device from the
// segment list this plan reports; the vnode's offset carries FT_KV_OFFSET_AUX.  A tail grows by one token per step
// of the burst: inside a group it is followed by tail_room spare entries, which no row attends to until the
// caller moves the row's range end.
struct Direct {
  int32_t tail_room = -1;
  const int64_t* node_base = nullptr;
  const int64_t* node_offset = nullptr;
  int64_t n_extra = 0;
  const int64_t* extra_begin = nullptr;
  const int64_t* extra_end = nullptr;
  const int32_t* extra_req = nullptr;
};

int build_plan(const int32_t* parent, const int32_t* seqlen, int32_t n_nodes, const int64_t* req_offs,
               const int32_t* req_ids, const int64_t* kv_ptrs, const Direct* direct, int32_t batch, int32_t num_qo_heads,
               int32_t num_kv_heads, int32_t head_dim, const ft_b200_model* model, ft_plan** out) {
  if (out == nullptr) return FT_ERR_INVALID_ARGUMENT;
  *out = nullptr;
  if (parent == nullptr || seqlen == nullptr || req_offs == nullptr || (kv_ptrs == nullptr && direct == nullptr) ||
      n_nodes <= 0 || batch < 0 || num_qo_heads <= 0 || num_kv_heads <= 0 || head_dim <= 0)
    return FT_ERR_INVALID_ARGUMENT;
  if (direct != nullptr &&
      (direct->node_base == nullptr || direct->node_offset == nullptr || direct->n_extra < 0 ||
       (direct->n_extra > 0 && (direct->extra_begin == nullptr || direct->extra_end == nullptr || direct->extra_req == nullptr))))
    return FT_ERR_INVALID_ARGUMENT;
  if (req_ids == nullptr && req_offs[n_nodes] > 0) return FT_ERR_INVALID_ARGUMENT;
  for (int i = 1; i < n_nodes; ++i)
    if (parent[i] < 0 || parent[i] >= i) return FT_ERR_INVALID_ARGUMENT;  // node 0 is the root, parents precede children
  Model m;
  if (model != nullptr) {
    m.num_sms = model->num_sms;
    m.ctas_per_sm = model->ctas_per_sm;
    m.waves = model->waves;
    m.tile_tokens = model->tile_tokens;
    m.rows_per_cta = model->rows_per_cta;
    m.min_chunk = model->min_chunk;
    m.nominal_split = model->nominal_split;
    m.ridge_flop_per_byte = model->ridge_flop_per_byte;
    m.task_overhead_bytes = model->task_overhead_bytes;
    m.elem_bytes = model->elem_bytes;
    m.group_member_tokens = model->group_member_tokens;
    m.group_min_members = model->group_min_members;
    if (m.group_member_tokens < 0 || m.group_min_members < 0) return FT_ERR_INVALID_ARGUMENT;
    if (m.num_sms <= 0 || m.ctas_per_sm <= 0 || !(m.waves > 0) || m.tile_tokens <= 0 || m.rows_per_cta <= 0 ||
        m.min_chunk <= 0 || m.nominal_split <= 0 || !(m.ridge_flop_per_byte > 0) || m.elem_bytes <= 0)
      return FT_ERR_INVALID_ARGUMENT;
  } else if (head_dim == 128) {
    m.rows_per_cta = 128;  // the tcgen05 stage-1 kernel holds 128 query rows per CTA
    m.ridge_flop_per_byte = 4 * m.ridge_flop_per_byte;
  }
  ft_plan* plan = new (std::nothrow) ft_plan();
  if (plan == nullptr) return FT_ERR_TOO_LARGE;
  try {
    const int n = n_nodes;
    const int group = std::max(1, num_qo_heads / num_kv_heads);
    const int q_tile = std::max(1, m.rows_per_cta / group);
    const int small_tile = std::max(1, std::min(q_tile, group <= 16 ? 16 / group : 1));
    auto n_req = [&](int i) { return req_offs[i + 1] - req_offs[i]; };

    // ---- 1. edges
    std::vector<std::vector<int>> kids(n);
    for (int i = 1; i < n; ++i) kids[parent[i]].push_back(i);
    std::vector<int64_t> run_len(seqlen, seqlen + n);
    std::vector<int32_t>& assign = plan->assignments;
    assign.assign(n, 0);
    // Per parent three candidates - the greedy walk over its children in id order, no child carrying, every child
    // carrying (the only one that removes the parent's own tasks) - and the cheapest wins (ties: greedy, then none).
    std::deque<int> frontier{0};
    std::vector<int> greedy;
    while (!frontier.empty()) {
      const int v = frontier.front();
      frontier.pop_front();
      if (kids[v].empty()) continue;
      const int64_t n_v = n_req(v), len_v = run_len[v];
      int64_t n_here = n_v;
      double greedy_cost = 0.0;
      greedy.clear();
      for (int c : kids[v]) {
        const int64_t n_c = n_req(c);
        const double own = task_cost(n_here, len_v, group, head_dim, m) + task_cost(n_c, run_len[c], group, head_dim, m);
        const double carried = task_cost(n_here - n_c, len_v, group, head_dim, m) +
                               task_cost(n_c, run_len[c] + len_v, group, head_dim, m);
        const bool take = carried < own;
        greedy.push_back(take ? 1 : 0);
        if (take) n_here -= n_c;
        greedy_cost += task_cost(n_c, run_len[c] + (take ? len_v : 0), group, head_dim, m);
      }
      greedy_cost += task_cost(n_here, len_v, group, head_dim, m);
      double none_cost = task_cost(n_v, len_v, group, head_dim, m), all_cost = 0.0;
      int64_t n_left = n_v;
      for (int c : kids[v]) {
        const int64_t n_c = n_req(c);
        none_cost += task_cost(n_c, run_len[c], group, head_dim, m);
        all_cost += task_cost(n_c, run_len[c] + len_v, group, head_dim, m);
        n_left -= n_c;
      }
      all_cost += task_cost(n_left, len_v, group, head_dim, m);  // requests that end at v itself keep its vnode
      int mode = 0;  // 0 greedy, 1 none, 2 all
      double best = greedy_cost;
      if (none_cost < best) mode = 1, best = none_cost;
      if (all_cost < best) mode = 2, best = all_cost;
      for (size_t k = 0; k < kids[v].size(); ++k) {
        const int c = kids[v][k];
        const bool take = mode == 2 || (mode == 0 && greedy[k] == 1);
        if (take) {
          assign[c] = 1;
          run_len[c] += len_v;
        }
        frontier.push_back(c);
      }
    }

    // ---- 2./3. virtual nodes: requests a node still serves, its row ranges, its chunk length
    struct Spec {
      std::vector<std::pair<int64_t, int64_t>> ranges;
      std::vector<int32_t> reqs;
      int64_t length;
      int64_t chunk;
      std::vector<std::pair<int32_t, int32_t>> row_ranges;  // group of short nodes: per request, its tokens of the chunk
      int64_t room = 0;                 // spare row ids kept behind this pairing when it becomes a member of a group
      std::vector<int64_t> member_room;  // group in the serving path: room behind each of its ranges
    };
    std::vector<Spec> specs;
    const int64_t row_bytes = 2LL * head_dim * m.elem_bytes;
    int64_t total_stream = 0;
    std::vector<uint8_t> gone((size_t)std::max(batch, 1));
    for (int i = 0; i < n; ++i) {
      // requests of this node minus those of children that carry its KV, sorted, duplicates removed
      std::vector<int32_t> reqs(req_ids + req_offs[i], req_ids + req_offs[i + 1]);
      std::sort(reqs.begin(), reqs.end());
      reqs.erase(std::unique(reqs.begin(), reqs.end()), reqs.end());
      for (int32_t r : reqs)
        if (r < 0 || r >= batch) {
          delete plan;
          return FT_ERR_INVALID_ARGUMENT;
        }
      bool any_gone = false;
      for (int c : kids[i])
        if (assign[c] == 1) {
          for (int64_t k = req_offs[c]; k < req_offs[c + 1]; ++k)
            if (req_ids[k] >= 0 && req_ids[k] < batch) gone[req_ids[k]] = 1, any_gone = true;
        }
      if (any_gone) {
        std::vector<int32_t> kept;
        for (int32_t r : reqs)
          if (!gone[r]) kept.push_back(r);
        for (int c : kids[i])
          if (assign[c] == 1)
            for (int64_t k = req_offs[c]; k < req_offs[c + 1]; ++k)
              if (req_ids[k] >= 0 && req_ids[k] < batch) gone[req_ids[k]] = 0;
        reqs.swap(kept);
      }
      if (reqs.empty()) continue;
      Spec s;
      if (direct != nullptr) {
        int top = i;
        while (assign[top] == 1) top = parent[top];
        s.ranges.emplace_back(direct->node_base[i] + direct->node_offset[top],
                              direct->node_base[i] + direct->node_offset[i] + seqlen[i]);
      } else {
        s.ranges.emplace_back(kv_ptrs[i], kv_ptrs[i + 1]);
        for (int up = i; assign[up] == 1;) {
          up = parent[up];
          s.ranges.emplace_back(kv_ptrs[up], kv_ptrs[up + 1]);
        }
        std::reverse(s.ranges.begin(), s.ranges.end());  // root-most segment first
      }
      s.length = 0;
      for (auto& r : s.ranges) s.length += r.second - r.first;
      if (s.length <= 0) continue;
      s.reqs.swap(reqs);
      total_stream += ceil_div((int64_t)s.reqs.size(), q_tile) * s.length * row_bytes;
      specs.push_back(std::move(s));
    }
    if (direct != nullptr) {
      for (int64_t e = 0; e < direct->n_extra; ++e) {
        const int64_t length = direct->extra_end[e] - direct->extra_begin[e];
        const int32_t r = direct->extra_req[e];
        if (r < 0 || r >= batch) {
          delete plan;
          return FT_ERR_INVALID_ARGUMENT;
        }
        if (length <= 0) continue;
        Spec s;
        s.ranges.emplace_back(direct->extra_begin[e], direct->extra_end[e]);
        s.reqs.push_back(r);
        s.length = length;
        s.room = std::max(direct->tail_room, 0);
        total_stream += ceil_div(1, q_tile) * length * row_bytes;
        specs.push_back(std::move(s));
      }
    }
    const double slots = (double)(m.num_sms * m.ctas_per_sm) * m.waves;
    const double target = std::max((double)(total_stream * num_kv_heads) / slots, (double)(m.min_chunk * row_bytes));
    for (Spec& s : specs) {
      const int64_t want = (int64_t)std::nearbyint((double)(s.length * row_bytes) / target);  // ties to even, like round()
      const int64_t n_chunks = std::max<int64_t>(1, std::min(want, ceil_div(s.length, m.min_chunk)));
      s.chunk = ceil_div(ceil_div(s.length, n_chunks), m.tile_tokens) * m.tile_tokens;
    }

    // ---- groups of short nodes (table-building mode, head_dim 128, 16-bit elements: the shape whose kernels honour
    // per-row token ranges).  Candidates - at most small_tile requests, at most group_member_tokens tokens - are
    // taken in order; a group is closed when the next candidate would exceed q_tile requests or 16 tiles of tokens,
    // would exceed the per-task token target (at least 4 tiles) once the group has more than small_tile requests,
    // or shares a request with it; groups with fewer than
    // group_min_members members, or not more requests than small_tile, are dissolved.  Result: the other virtual
    // nodes in their order, then groups and dissolved candidates in the order they were closed.
    bool any_groups = false;
    if ((direct == nullptr || direct->tail_room >= 0) && head_dim == 128 && m.elem_bytes == 2 && m.group_member_tokens > 0) {
      const int64_t tile = m.tile_tokens;
      const int64_t target_tokens = (int64_t)std::floor(target / (double)row_bytes);
      int64_t hard_cap = 16 * tile;
      int64_t cap = std::min(std::max(target_tokens / tile * tile, 4 * tile), hard_cap);
      if (direct != nullptr) {
        // Serving path: the groups are sized so that the step fills two rounds of resident CTAs, the other tasks
        // included (measured: their tiles are gathered row by row, and two shorter groups per slot hide that latency
        // better than one long one, while a third round costs more than it hides), up to 24 tiles.
        int64_t cand_tokens = 0, other = 0;
        for (const Spec& s : specs) {
          const int64_t nreq = (int64_t)s.reqs.size();
          if (nreq <= small_tile && s.length + s.room <= m.group_member_tokens) cand_tokens += s.length + s.room;
          else other += ceil_div(s.length, s.chunk) * ceil_div(nreq, q_tile);
        }
        const int64_t round = std::max<int64_t>((int64_t)slots / std::max(num_kv_heads, 1), 1);
        const int64_t free_tasks = std::max<int64_t>(std::max(2 * round - other, round / 2), 2);
        hard_cap = 24 * tile;
        cap = std::min(std::max(ceil_div(ceil_div(cand_tokens, free_tasks), tile) * tile, 4 * tile), hard_cap);
      }
      else {
        // One round: when the tasks at the default cap would spill a little past one round of resident CTAs while
        // longer groups keep everything inside it, the cap grows to what fills the round exactly.
        int64_t cand_tokens = 0, other = 0;
        for (const Spec& s : specs) {
          const int64_t nreq = (int64_t)s.reqs.size();
          if (nreq <= small_tile && s.length <= m.group_member_tokens) cand_tokens += s.length;
          else other += ceil_div(s.length, s.chunk) * ceil_div(nreq, q_tile);
        }
        const int64_t round = std::max<int64_t>((int64_t)(m.num_sms * m.ctas_per_sm) / std::max(num_kv_heads, 1), 1);
        if (other < round && other + ceil_div(cand_tokens, cap) > round) {
          const int64_t fill = ceil_div(ceil_div(cand_tokens, round - other), tile) * tile;
          if (fill <= hard_cap) cap = std::max(cap, fill);
        }
      }
      std::vector<Spec> kept, tail;
      std::vector<Spec> cur;
      std::vector<uint8_t> in_group((size_t)std::max(batch, 1), 0);
      int64_t cur_tokens = 0, cur_n = 0;
      auto close = [&]() {
        for (const Spec& c : cur)
          for (int32_t r : c.reqs) in_group[r] = 0;
        if ((int64_t)cur.size() >= m.group_min_members && cur_n > small_tile) {
          Spec g;
          int64_t start = 0;
          for (Spec& c : cur) {
            g.ranges.insert(g.ranges.end(), c.ranges.begin(), c.ranges.end());
            g.reqs.insert(g.reqs.end(), c.reqs.begin(), c.reqs.end());
            g.row_ranges.insert(g.row_ranges.end(), c.reqs.size(), std::make_pair((int32_t)start, (int32_t)(start + c.length)));
            if (direct != nullptr) g.member_room.push_back(c.room);  // one range per member in the serving path
            start += c.length + c.room;
          }
          g.length = start;
          g.chunk = ceil_div(start, tile) * tile;
          tail.push_back(std::move(g));
          any_groups = true;
        } else {
          for (Spec& c : cur) tail.push_back(std::move(c));
        }
        cur.clear();
        cur_tokens = cur_n = 0;
      };
      for (Spec& s : specs) {
        const int64_t nreq = (int64_t)s.reqs.size();
        const int64_t span = s.length + s.room;
        if (nreq <= small_tile && span <= m.group_member_tokens) {
          bool shared = false;
          for (int32_t r : s.reqs) shared = shared || in_group[r] != 0;
          // (serving path: a group is closed once it has reached the cap, not before it would pass it, so that
          // the groups number no more than the tasks they were sized for)
          const bool full = direct != nullptr ? cur_tokens >= cap : cur_tokens + span > cap;
          if (!cur.empty() && (cur_n + nreq > q_tile || cur_tokens + span > hard_cap || (full && cur_n > small_tile) || shared))
            close();
          for (int32_t r : s.reqs) in_group[r] = 1;
          cur_tokens += span;
          cur_n += nreq;
          cur.push_back(std::move(s));
        } else {
          kept.push_back(std::move(s));
        }
      }
      close();
      specs.swap(kept);
      for (Spec& t : tail) specs.push_back(std::move(t));
    }

    // ---- tail split (table-building mode).  The hardware hands CTAs to slots in grid order, so a step of 2.05 or 2.6
    // rounds ends with a round in which a fraction of the slots run whole tasks while the rest of the GPU idles.  On a
    // simulated list schedule of the tasks in emission order (integer time: a fixed cost per task plus one unit per
    // KV tile; a task = the CTAs of all KV heads of one chunk x request tile, which start side by side), when the
    // makespan exceeds the perfectly packed time by more than an eighth, every plain (ungrouped) virtual node with a
    // task that ends in the later half of that excess is cut to half its chunk length (never below min_chunk); the
    // cut is kept if the simulated makespan drops.  (A step of one round lasts as long as its longest task: same cut.)
    if (direct == nullptr) {
      const int64_t start_cost[2] = {5, 4};  // many-row / few-row task, in tile times
      const int64_t sched_slots = std::max<int64_t>((int64_t)(m.num_sms * m.ctas_per_sm) / std::max(num_kv_heads, 1), 1);
      struct SimTask {
        int phase;
        int64_t key, seq, dur;
        size_t spec;
      };
      auto simulate = [&](const std::vector<int64_t>& chunk_of, std::vector<int64_t>& last_end, int64_t& total) {
        std::vector<SimTask> tasks;
        for (size_t si = 0; si < specs.size(); ++si) {
          const Spec& s = specs[si];
          const int64_t nreq = (int64_t)s.reqs.size();
          if (nreq == 0 || s.length <= 0) continue;
          const int64_t n_kv = ceil_div(s.length, chunk_of[si]), n_q = ceil_div(nreq, q_tile);
          for (int64_t c = 0; c < n_kv; ++c) {
            const int64_t c_len = std::min((c + 1) * chunk_of[si], s.length) - c * chunk_of[si];
            for (int64_t t = 0; t < n_q; ++t) {
              const int64_t q_len = std::min((t + 1) * (int64_t)q_tile, nreq) - t * q_tile;
              const int phase = q_len > small_tile ? 0 : 1;
              tasks.push_back({phase, c_len * 64 + std::min<int64_t>(q_len, 63), (int64_t)tasks.size(),
                               start_cost[phase] + ceil_div(c_len, m.tile_tokens), si});
            }
          }
        }
        std::stable_sort(tasks.begin(), tasks.end(), [](const SimTask& a, const SimTask& b) {
          return a.phase != b.phase ? a.phase < b.phase : a.key > b.key;
        });
        std::priority_queue<int64_t, std::vector<int64_t>, std::greater<int64_t>> free_at;
        for (int64_t k = 0; k < sched_slots; ++k) free_at.push(0);
        last_end.assign(specs.size(), 0);
        int64_t makespan = 0;
        total = 0;
        for (const SimTask& t : tasks) {
          const int64_t start = free_at.top();
          free_at.pop();
          free_at.push(start + t.dur);
          last_end[t.spec] = std::max(last_end[t.spec], start + t.dur);
          makespan = std::max(makespan, start + t.dur);
          total += t.dur;
        }
        return makespan;
      };
      std::vector<int64_t> chunk_of(specs.size()), last_end;
      for (size_t si = 0; si < specs.size(); ++si) chunk_of[si] = specs[si].chunk;
      int64_t total = 0;
      const int64_t makespan = simulate(chunk_of, last_end, total);
      const int64_t bound = ceil_div(total, sched_slots);
      if ((makespan - bound) * 8 > makespan) {
        const int64_t late_from = makespan - (makespan - bound + 1) / 2;
        std::vector<int64_t> trial(chunk_of);
        bool any = false;
        for (size_t si = 0; si < specs.size(); ++si) {
          const Spec& s = specs[si];
          if (!s.row_ranges.empty() || last_end[si] <= late_from) continue;
          const int64_t cur = std::min(chunk_of[si], s.length);
          const int64_t half = ceil_div(ceil_div(cur, 2), m.tile_tokens) * m.tile_tokens;
          if (half >= m.min_chunk && half < cur) {
            trial[si] = half;
            any = true;
          }
        }
        if (any) {
          std::vector<int64_t> fs2;
          int64_t total2 = 0;
          if (simulate(trial, fs2, total2) < makespan)
            for (size_t si = 0; si < specs.size(); ++si) specs[si].chunk = trial[si];
        }
      }
    }

    // ---- emission: chunk-major, request-tile-minor; every chunk repeats the node's request list
    std::vector<int64_t> kv_offs, kv_lens, q_offs, q_lens;
    int64_t kv_total = 0, q_total = 0, aux_total = 0;
    for (const Spec& s : specs) {
      const int64_t nreq = (int64_t)s.reqs.size();
      int64_t kv_base = direct != nullptr ? s.ranges[0].first : kv_total;
      if (direct != nullptr && !s.member_room.empty()) {  // a group of the serving path: its row ids live in the auxiliary table
        kv_base = (int64_t)FT_KV_OFFSET_AUX + aux_total;
        int64_t at = aux_total;
        for (size_t k = 0; k < s.ranges.size(); ++k) {
          const int64_t len = s.ranges[k].second - s.ranges[k].first;
          if (s.ranges[k].first >= (int64_t)FT_KV_OFFSET_AUX || at + len + s.member_room[k] >= (int64_t)FT_KV_OFFSET_AUX) {
            delete plan;
            return FT_ERR_TOO_LARGE;
          }
          plan->aux_segments.push_back((int32_t)s.ranges[k].first);
          plan->aux_segments.push_back((int32_t)len);
          plan->aux_segments.push_back((int32_t)at);
          plan->aux_segments.push_back((int32_t)s.member_room[k]);
          at += len + s.member_room[k];
        }
        aux_total = at;
      }
      if (direct == nullptr)
        for (auto& r : s.ranges)
          for (int64_t row = r.first; row < r.second; ++row) plan->kv_entries.push_back((int32_t)row);
      const int64_t n_kv = ceil_div(s.length, s.chunk), n_q = ceil_div(nreq, q_tile);
      for (int64_t c = 0; c < n_kv; ++c) {
        const int64_t c_off = c * s.chunk, c_len = std::min(c_off + s.chunk, s.length) - c_off;
        for (int64_t t = 0; t < n_q; ++t) {
          const int64_t t_off = t * q_tile;
          kv_offs.push_back(kv_base + c_off);
          kv_lens.push_back(c_len);
          q_offs.push_back(q_total + c * nreq + t_off);
          q_lens.push_back(std::min(t_off + q_tile, nreq) - t_off);
        }
        plan->q_entries.insert(plan->q_entries.end(), s.reqs.begin(), s.reqs.end());
        if (any_groups) {
          for (int64_t r = 0; r < nreq; ++r) {
            plan->q_ranges.push_back(s.row_ranges.empty() ? 0 : s.row_ranges[(size_t)r].first);
            // a row of a plain vnode sees its whole chunk; in the serving path that chunk may grow during the burst
            // (vnode_to_kv_lens is bumped), so the end is left open there - the kernels clip it to the chunk
            plan->q_ranges.push_back(s.row_ranges.empty() ? (direct != nullptr ? INT32_MAX : (int32_t)c_len)
                                                          : s.row_ranges[(size_t)r].second);
          }
        }
      }
      kv_total += s.length;
      q_total += n_kv * nreq;
    }
    const int64_t pad = 32;  // the reference appends 32 x -1 to both index lists (fasttree.py:261-262)
    int64_t max_off = 0;
    for (int64_t o : kv_offs) max_off = std::max(max_off, o);
    if (kv_total + pad >= (1LL << 31) || q_total >= (1LL << 31) || max_off >= (1LL << 31)) {
      delete plan;
      return FT_ERR_TOO_LARGE;
    }
    if (direct == nullptr) plan->kv_entries.insert(plan->kv_entries.end(), (size_t)pad, -1);

    // request -> partial rows: rows grouped by request id, emission order kept inside a group
    std::vector<int64_t> counts((size_t)batch, 0);
    for (int32_t r : plan->q_entries) ++counts[r];
    plan->r2v_offs.resize(batch);
    plan->r2v_lens.resize(batch);
    int64_t acc = 0;
    for (int b = 0; b < batch; ++b) {
      plan->r2v_offs[b] = (int32_t)acc;
      plan->r2v_lens[b] = (int32_t)counts[b];
      acc += counts[b];
    }
    plan->r2v_entries.assign((size_t)(q_total + pad), -1);
    {
      std::vector<int64_t> cursor(plan->r2v_offs.begin(), plan->r2v_offs.end());
      for (int64_t row = 0; row < q_total; ++row) plan->r2v_entries[(size_t)cursor[plan->q_entries[row]]++] = (int32_t)row;
    }

    // phases and order: more requests than the small tile first; inside a phase longest KV chunk first, then
    // more requests first (key = kv_len * 64 + min(q_len, 63)), stable
    const size_t nv = kv_offs.size();
    std::vector<size_t> big, small;
    for (size_t i = 0; i < nv; ++i) (q_lens[i] > small_tile ? big : small).push_back(i);
    auto key = [&](size_t i) { return kv_lens[i] * 64 + std::min<int64_t>(q_lens[i], 63); };
    auto by_key = [&](size_t a, size_t b) { return key(a) > key(b); };
    std::stable_sort(big.begin(), big.end(), by_key);
    std::stable_sort(small.begin(), small.end(), by_key);
    std::vector<size_t> perm(big);
    perm.insert(perm.end(), small.begin(), small.end());
    plan->kv_offs.resize(nv);
    plan->kv_lens.resize(nv);
    plan->q_offs.resize(nv);
    plan->q_lens.resize(nv);
    for (size_t i = 0; i < nv; ++i) {
      plan->kv_offs[i] = (int32_t)kv_offs[perm[i]];
      plan->kv_lens[i] = (int32_t)kv_lens[perm[i]];
      plan->q_offs[i] = (int32_t)q_offs[perm[i]];
      plan->q_lens[i] = (int32_t)q_lens[perm[i]];
    }
    ft_plan_info& info = plan->info;
    std::memset(&info, 0, sizeof(info));
    info.kv_entries = (int64_t)plan->kv_entries.size();
    info.vnodes = (int64_t)nv;
    info.partial_rows = q_total;
    info.batch = batch;
    info.nodes = n;
    info.phase_node_nums[0] = (int32_t)big.size();
    info.phase_node_nums[1] = (int32_t)small.size();
    info.phase_node_offsets[0] = 0;
    info.phase_node_offsets[1] = (int32_t)big.size();
    info.q_tile = q_tile;
    info.small_tile = small_tile;
    info.tile_tokens = m.tile_tokens;
    info.has_row_ranges = any_groups ? 1 : 0;
    info.aux_entries = aux_total;
    info.aux_segments = (int64_t)(plan->aux_segments.size() / 4);
    info.target_bytes = target;
    info.virtual_nodes = (int64_t)specs.size();
  } catch (const std::bad_alloc&) {
    delete plan;
    return FT_ERR_TOO_LARGE;
  }
  *out = plan;
  return FT_OK;
}

}  // namespace

extern "C" {

int ft_plan_b200_build(const int32_t* parent, const int32_t* seqlen, int32_t n_nodes, const int64_t* req_offs,
                       const int32_t* req_ids, const int64_t* kv_ptrs, int32_t batch, int32_t num_qo_heads,
                       int32_t num_kv_heads, int32_t head_dim, const ft_b200_model* model, ft_plan** out) {
  return build_plan(parent, seqlen, n_nodes, req_offs, req_ids, kv_ptrs, nullptr, batch, num_qo_heads, num_kv_heads,
                    head_dim, model, out);
}

int ft_plan_b200_build_direct(const int32_t* parent, const int32_t* seqlen, int32_t n_nodes, const int64_t* req_offs,
                              const int32_t* req_ids, const int64_t* node_base, const int64_t* node_offset,
                              int64_t n_extra, const int64_t* extra_begin, const int64_t* extra_end,
                              const int32_t* extra_req, int32_t tail_room, int32_t batch, int32_t num_qo_heads,
                              int32_t num_kv_heads, int32_t head_dim, const ft_b200_model* model, ft_plan** out) {
  Direct d;
  d.tail_room = tail_room;
  d.node_base = node_base;
  d.node_offset = node_offset;
  d.n_extra = n_extra;
  d.extra_begin = extra_begin;
  d.extra_end = extra_end;
  d.extra_req = extra_req;
  return build_plan(parent, seqlen, n_nodes, req_offs, req_ids, nullptr, &d, batch, num_qo_heads, num_kv_heads, head_dim,
                    model, out);
}

int ft_plan_get_info(const ft_plan* plan, ft_plan_info* info) {
  if (plan == nullptr || info == nullptr) return FT_ERR_INVALID_ARGUMENT;
  *info = plan->info;
  return FT_OK;
}

// Copies the tables into caller-provided host arrays of the sizes ft_plan_get_info reports (NULL: skip that table).
int ft_plan_copy_tables(const ft_plan* plan, int32_t* kv_entries, int32_t* kv_offs, int32_t* kv_lens, int32_t* q_entries,
                        int32_t* q_offs, int32_t* q_lens, int32_t* r2v_entries, int32_t* r2v_offs, int32_t* r2v_lens,
                        int32_t* node_assignments) {
  if (plan == nullptr) return FT_ERR_INVALID_ARGUMENT;
  auto put = [](int32_t* dst, const std::vector<int32_t>& src) {
    if (dst != nullptr && !src.empty()) std::memcpy(dst, src.data(), src.size() * sizeof(int32_t));
  };
  put(kv_entries, plan->kv_entries);
  put(kv_offs, plan->kv_offs);
  put(kv_lens, plan->kv_lens);
  put(q_entries, plan->q_entries);
  put(q_offs, plan->q_offs);
  put(q_lens, plan->q_lens);
  put(r2v_entries, plan->r2v_entries);
  put(r2v_offs, plan->r2v_offs);
  put(r2v_lens, plan->r2v_lens);
  put(node_assignments, plan->assignments);
  return FT_OK;
}

int ft_plan_copy_row_ranges(const ft_plan* plan, int32_t* q_kv_ranges) {
  if (plan == nullptr || q_kv_ranges == nullptr || plan->q_ranges.empty()) return FT_ERR_INVALID_ARGUMENT;
  std::memcpy(q_kv_ranges, plan->q_ranges.data(), plan->q_ranges.size() * sizeof(int32_t));
  return FT_OK;
}

int ft_plan_copy_aux_segments(const ft_plan* plan, int32_t* segments) {
  if (plan == nullptr || segments == nullptr || plan->aux_segments.empty()) return FT_ERR_INVALID_ARGUMENT;
  std::memcpy(segments, plan->aux_segments.data(), plan->aux_segments.size() * sizeof(int32_t));
  return FT_OK;
}

void ft_plan_free(ft_plan* plan) { delete plan; }

}  // extern "C"
