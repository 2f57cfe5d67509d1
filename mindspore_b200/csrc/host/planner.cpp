// Host-side planners: pipeline schedules, static memory planning, strategy search.
//
//  * msb_pipeline_schedule   - per-stage order of forward/backward micro-batch steps for GPipe, 1F1B and
//    interleaved 1F1B (several model chunks per stage).  Role of the reference's pipeline scheduler
//    (ccsrc/frontend/parallel/pipeline_transformer/pipeline_scheduler.cc:251-771), re-expressed as a step list the
//    runtime executes instead of a graph reordering.
//  * msb_memory_plan         - lifetime-aware offset assignment (best-fit over live intervals) so that a
//    compiled graph runs out of one arena; contiguity groups keep fused-communication members adjacent.
//    Role of SOMAS (ccsrc/backend/common/somas/somas.cc, somas_solver_*.cc).
//  * msb_chain_dp_search     - exact dynamic programming over a chain of operators choosing one strategy per
//    operator to minimise compute + redistribution cost (the core recurrence of the reference's DP search,
//    ccsrc/frontend/parallel/auto_parallel/dp_algo_costmodel.cc, restricted to chains).
//  * msb_propagate_strategies- sharding propagation on a DAG: strategies fixed by the user spread to neighbours
//    by picking, per edge, the candidate with the least redistribution cost
//    (ccsrc/frontend/parallel/auto_parallel/graph_costmodel.cc:196-319).
#include <algorithm>
#include <cstdint>
#include <deque>
#include <limits>
#include <map>
#include <vector>

#define MSB_API extern "C" __attribute__((visibility("default")))

// ------------------------------------------------------------------------------------------------ pipeline
// out: 3 ints per step {kind (0 forward, 1 backward), micro_batch, chunk}.  scheduler: 0 GPipe, 1 1F1B.
// chunks > 1 selects the interleaved schedule (virtual stages): model chunk c of stage s is virtual stage
// c*stages + s.  Returns the number of steps, -1 if capacity is too small, -2 on invalid arguments.
MSB_API int msb_pipeline_schedule(int stages, int stage, int micro, int chunks, int scheduler, int32_t* out,
                                  int capacity) {
  if (stages < 1 || stage < 0 || stage >= stages || micro < 1 || chunks < 1) return -2;
  if (chunks > 1 && micro % stages != 0) return -2;  // interleaved 1F1B needs micro to be a multiple of stages
  std::vector<int32_t> steps;
  auto push = [&](int kind, int mb, int chunk) {
    steps.push_back(kind);
    steps.push_back(mb);
    steps.push_back(chunk);
  };
  const int total = micro * chunks;
  // order in which (micro, chunk) pairs are visited by forward steps on one stage
  auto fwd_at = [&](int i, int& mb, int& chunk) {
    if (chunks == 1) { mb = i; chunk = 0; return; }
    const int group = i / (stages * chunks);
    const int in_group = i % (stages * chunks);
    chunk = in_group / stages;
    mb = group * stages + in_group % stages;
  };
  auto bwd_at = [&](int i, int& mb, int& chunk) {
    if (chunks == 1) { mb = i; chunk = 0; return; }
    const int group = i / (stages * chunks);
    const int in_group = i % (stages * chunks);
    chunk = chunks - 1 - in_group / stages;
    mb = group * stages + in_group % stages;
  };
  if (scheduler == 0) {
    for (int i = 0; i < total; ++i) { int mb, c; fwd_at(i, mb, c); push(0, mb, c); }
    for (int i = 0; i < total; ++i) { int mb, c; bwd_at(i, mb, c); push(1, mb, c); }
  } else {
    int warmup;
    if (chunks == 1) {
      warmup = std::min(stages - stage - 1, total);
    } else {
      warmup = std::min((stages - stage - 1) * 2 + (chunks - 1) * stages, total);
    }
    int f = 0, b = 0;
    for (int i = 0; i < warmup; ++i, ++f) { int mb, c; fwd_at(f, mb, c); push(0, mb, c); }
    while (f < total) {
      int mb, c;
      fwd_at(f++, mb, c); push(0, mb, c);
      bwd_at(b++, mb, c); push(1, mb, c);
    }
    while (b < total) { int mb, c; bwd_at(b++, mb, c); push(1, mb, c); }
  }
  const int n = static_cast<int>(steps.size() / 3);
  if (n > capacity) return -1;
  std::copy(steps.begin(), steps.end(), out);
  return n;
}

// Peak number of micro-batches whose activations are alive on `stage` under the schedule.
MSB_API int msb_pipeline_peak_activations(const int32_t* steps, int n) {
  int live = 0, peak = 0;
  for (int i = 0; i < n; ++i) {
    live += steps[3 * i] == 0 ? 1 : -1;
    peak = std::max(peak, live);
  }
  return peak;
}

// ------------------------------------------------------------------------------------------------ memory plan
// Tensor i lives during [start[i], end[i]] (inclusive step indices) and needs size[i] bytes.  group[i] >= 0
// marks members of a contiguity group (laid out back to back in index order); -1 = free-standing.
// offsets_out[i] receives the arena offset.  Returns the arena size (<0 on error).
MSB_API int64_t msb_memory_plan(int n, const int64_t* size, const int32_t* start, const int32_t* end,
                                const int32_t* group, int64_t align, int64_t* offsets_out) {
  if (n < 0 || align <= 0) return -1;
  struct Block { int64_t size; int32_t s, e; std::vector<int> members; };
  std::vector<Block> blocks;
  std::map<int, int> group_block;
  auto up = [&](int64_t v) { return (v + align - 1) / align * align; };
  for (int i = 0; i < n; ++i) {
    if (end[i] < start[i] || size[i] < 0) return -1;
    const int g = group ? group[i] : -1;
    if (g >= 0) {
      auto it = group_block.find(g);
      if (it == group_block.end()) {
        group_block[g] = static_cast<int>(blocks.size());
        blocks.push_back({up(size[i]), start[i], end[i], {i}});
      } else {
        Block& b = blocks[it->second];
        b.size += up(size[i]);
        b.s = std::min(b.s, start[i]);
        b.e = std::max(b.e, end[i]);
        b.members.push_back(i);
      }
    } else {
      blocks.push_back({up(size[i]), start[i], end[i], {i}});
    }
  }
  std::vector<int> order(blocks.size());
  for (size_t i = 0; i < order.size(); ++i) order[i] = static_cast<int>(i);
  // big and long-lived first
  std::sort(order.begin(), order.end(), [&](int a, int b) {
    if (blocks[a].size != blocks[b].size) return blocks[a].size > blocks[b].size;
    return (blocks[a].e - blocks[a].s) > (blocks[b].e - blocks[b].s);
  });
  std::vector<int64_t> block_off(blocks.size(), -1);
  std::vector<int> placed;
  int64_t arena = 0;
  for (int bi : order) {
    const Block& b = blocks[bi];
    std::vector<std::pair<int64_t, int64_t>> busy;  // [off, off+size) of overlapping-lifetime blocks
    for (int pj : placed) {
      const Block& o = blocks[pj];
      if (o.s <= b.e && b.s <= o.e) busy.emplace_back(block_off[pj], block_off[pj] + o.size);
    }
    std::sort(busy.begin(), busy.end());
    int64_t best = -1, best_gap = std::numeric_limits<int64_t>::max(), cursor = 0;
    for (auto& iv : busy) {
      if (iv.first - cursor >= b.size && iv.first - cursor < best_gap) {
        best = cursor;
        best_gap = iv.first - cursor;
      }
      cursor = std::max(cursor, iv.second);
    }
    if (best < 0) best = cursor;
    block_off[bi] = best;
    arena = std::max(arena, best + b.size);
    placed.push_back(bi);
  }
  for (size_t bi = 0; bi < blocks.size(); ++bi) {
    int64_t off = block_off[bi];
    for (int m : blocks[bi].members) {
      offsets_out[m] = off;
      off += up(size[m]);
    }
  }
  return arena;
}

// Verifies a plan: returns the number of pairs that overlap in both time and address range (0 = valid).
MSB_API int msb_memory_plan_check(int n, const int64_t* size, const int32_t* start, const int32_t* end,
                                  const int64_t* offsets) {
  int bad = 0;
  for (int i = 0; i < n; ++i)
    for (int j = i + 1; j < n; ++j)
      if (start[i] <= end[j] && start[j] <= end[i] && size[i] > 0 && size[j] > 0 &&
          offsets[i] < offsets[j] + size[j] && offsets[j] < offsets[i] + size[i])
        ++bad;
  return bad;
}

// ------------------------------------------------------------------------------------------------ strategy search
// Chain DP: operator t has n_cand[t] candidate strategies with compute cost op_cost[off_t + s]; moving from
// candidate a of op t to candidate b of op t+1 costs edge_cost[edge_off_t + a*n_cand[t+1] + b].
// choice_out[t] = selected candidate.  Returns the minimal total cost.
MSB_API double msb_chain_dp_search(int n_ops, const int32_t* n_cand, const double* op_cost, const double* edge_cost,
                                   int32_t* choice_out) {
  if (n_ops <= 0) return 0.0;
  std::vector<int> op_off(n_ops + 1, 0), edge_off(n_ops, 0);
  for (int t = 0; t < n_ops; ++t) op_off[t + 1] = op_off[t] + n_cand[t];
  for (int t = 0; t + 1 < n_ops; ++t) edge_off[t + 1] = edge_off[t] + n_cand[t] * n_cand[t + 1];
  std::vector<std::vector<double>> best(n_ops);
  std::vector<std::vector<int>> from(n_ops);
  best[0].assign(op_cost + op_off[0], op_cost + op_off[1]);
  from[0].assign(n_cand[0], -1);
  for (int t = 1; t < n_ops; ++t) {
    best[t].assign(n_cand[t], std::numeric_limits<double>::infinity());
    from[t].assign(n_cand[t], -1);
    for (int b = 0; b < n_cand[t]; ++b)
      for (int a = 0; a < n_cand[t - 1]; ++a) {
        const double c = best[t - 1][a] + edge_cost[edge_off[t - 1] + a * n_cand[t] + b] + op_cost[op_off[t] + b];
        if (c < best[t][b]) { best[t][b] = c; from[t][b] = a; }
      }
  }
  int cur = static_cast<int>(std::min_element(best[n_ops - 1].begin(), best[n_ops - 1].end()) - best[n_ops - 1].begin());
  const double total = best[n_ops - 1][cur];
  for (int t = n_ops - 1; t >= 0; --t) {
    choice_out[t] = cur;
    cur = from[t][cur];
  }
  return total;
}

// Sharding propagation.  Nodes 0..n-1; fixed[i] >= 0 pins node i to that candidate.  Edges (src[e], dst[e]);
// edge_cost for edge e is a dense [n_cand[src] x n_cand[dst]] block starting at cost_off[e].
// Breadth-first from the pinned nodes; an unvisited neighbour takes the candidate with the least cost on the
// connecting edge (ties: lowest index).  Nodes not reachable from a pinned node get candidate 0.
MSB_API int msb_propagate_strategies(int n, const int32_t* n_cand, const int32_t* fixed, int n_edges,
                                     const int32_t* src, const int32_t* dst, const int64_t* cost_off,
                                     const double* edge_cost, int32_t* choice_out) {
  std::vector<std::vector<std::pair<int, int>>> adj(n);  // (neighbour, edge index; sign encodes direction)
  for (int e = 0; e < n_edges; ++e) {
    if (src[e] < 0 || src[e] >= n || dst[e] < 0 || dst[e] >= n) return -1;
    adj[src[e]].emplace_back(dst[e], e + 1);
    adj[dst[e]].emplace_back(src[e], -(e + 1));
  }
  std::deque<int> queue;
  for (int i = 0; i < n; ++i) {
    choice_out[i] = -1;
    if (fixed[i] >= 0) {
      if (fixed[i] >= n_cand[i]) return -1;
      choice_out[i] = fixed[i];
      queue.push_back(i);
    }
  }
  int assigned = 0;
  while (!queue.empty()) {
    const int u = queue.front();
    queue.pop_front();
    for (auto& pr : adj[u]) {
      const int v = pr.first;
      if (choice_out[v] >= 0) continue;
      const bool forward = pr.second > 0;
      const int e = std::abs(pr.second) - 1;
      const double* block = edge_cost + cost_off[e];
      int best = 0;
      double best_cost = std::numeric_limits<double>::infinity();
      for (int c = 0; c < n_cand[v]; ++c) {
        const double cost = forward ? block[choice_out[u] * n_cand[v] + c] : block[c * n_cand[u] + choice_out[u]];
        if (cost < best_cost) { best_cost = cost; best = c; }
      }
      choice_out[v] = best;
      ++assigned;
      queue.push_back(v);
    }
  }
  for (int i = 0; i < n; ++i)
    if (choice_out[i] < 0) choice_out[i] = 0;
  return assigned;
}

// ------------------------------------------------------------------------------------------------ elimination search
// Exact minimum of   sum_i op_cost[i][c_i] + sum_e edge_cost[e][c_src][c_dst]   over all assignments, by eliminating
// the nodes one after the other (min-degree order): removing node v folds its own cost and every cost table that
// mentions v into one table over v's remaining neighbours, remembering the best candidate of v for each of their
// assignments.  Eliminating a node of degree 1 / 2 / 3 is what the reference calls operator, edge / merge /
// contract, and triangle / star elimination (auto_parallel/graph_costmodel.cc:866-1776, dp_algo_costmodel.cc); the
// general form handles any graph whose neighbourhoods stay small.  fixed[i] >= 0 pins node i.
// Returns the optimal cost, or -1 when a table would exceed `max_table` entries (caller falls back).
namespace {
struct Factor {
  std::vector<int> vars;
  std::vector<double> tab;   // row-major over vars, last var fastest
};
}  // namespace

MSB_API double msb_elimination_search(int n, const int32_t* n_cand, const double* op_cost, int n_edges,
                                      const int32_t* src, const int32_t* dst, const int64_t* cost_off,
                                      const double* edge_cost, const int32_t* fixed, long long max_table,
                                      int32_t* choice_out) {
  const double INF = std::numeric_limits<double>::infinity();
  if (n <= 0) return 0.0;
  std::vector<int> op_off(n + 1, 0);
  for (int i = 0; i < n; ++i) op_off[i + 1] = op_off[i] + n_cand[i];
  std::vector<Factor> factors;
  for (int i = 0; i < n; ++i) {
    Factor f;
    f.vars = {i};
    f.tab.assign(op_cost + op_off[i], op_cost + op_off[i + 1]);
    if (fixed && fixed[i] >= 0)
      for (int c = 0; c < n_cand[i]; ++c)
        if (c != fixed[i]) f.tab[c] = INF;
    factors.push_back(std::move(f));
  }
  for (int e = 0; e < n_edges; ++e) {
    if (src[e] < 0 || src[e] >= n || dst[e] < 0 || dst[e] >= n || src[e] == dst[e]) return -1;
    Factor f;
    f.vars = {src[e], dst[e]};
    f.tab.assign(edge_cost + cost_off[e], edge_cost + cost_off[e] + static_cast<long long>(n_cand[src[e]]) * n_cand[dst[e]]);
    factors.push_back(std::move(f));
  }
  std::vector<bool> alive_f(factors.size(), true), gone(n, false);
  struct Decision {
    int var;
    std::vector<int> scope;
    std::vector<int32_t> arg;
  };
  std::vector<Decision> decisions;
  double constant = 0.0;
  for (int step = 0; step < n; ++step) {
    // interaction-graph degree of every remaining node
    int best_v = -1;
    size_t best_deg = static_cast<size_t>(-1);
    for (int v = 0; v < n; ++v) {
      if (gone[v]) continue;
      std::vector<int> nb;
      for (size_t fi = 0; fi < factors.size(); ++fi) {
        if (!alive_f[fi]) continue;
        const auto& vs = factors[fi].vars;
        if (std::find(vs.begin(), vs.end(), v) == vs.end()) continue;
        for (int u : vs)
          if (u != v && std::find(nb.begin(), nb.end(), u) == nb.end()) nb.push_back(u);
      }
      if (nb.size() < best_deg) { best_deg = nb.size(); best_v = v; }
    }
    const int v = best_v;
    std::vector<size_t> mine;
    std::vector<int> scope;
    for (size_t fi = 0; fi < factors.size(); ++fi) {
      if (!alive_f[fi]) continue;
      const auto& vs = factors[fi].vars;
      if (std::find(vs.begin(), vs.end(), v) == vs.end()) continue;
      mine.push_back(fi);
      for (int u : vs)
        if (u != v && std::find(scope.begin(), scope.end(), u) == scope.end()) scope.push_back(u);
    }
    std::sort(scope.begin(), scope.end());
    long long size = 1;
    for (int u : scope) {
      size *= n_cand[u];
      if (size > max_table) return -1;
    }
    Factor nf;
    nf.vars = scope;
    nf.tab.assign(static_cast<size_t>(size), INF);
    Decision d;
    d.var = v;
    d.scope = scope;
    d.arg.assign(static_cast<size_t>(size), 0);
    std::vector<int> assign(n, 0);
    for (long long idx = 0; idx < size; ++idx) {
      long long rem = idx;
      for (int k = static_cast<int>(scope.size()) - 1; k >= 0; --k) {
        assign[scope[k]] = static_cast<int>(rem % n_cand[scope[k]]);
        rem /= n_cand[scope[k]];
      }
      double best = INF;
      int best_c = 0;
      for (int c = 0; c < n_cand[v]; ++c) {
        assign[v] = c;
        double sum = 0.0;
        for (size_t fi : mine) {
          const Factor& f = factors[fi];
          long long off = 0;
          for (int u : f.vars) off = off * n_cand[u] + assign[u];
          sum += f.tab[static_cast<size_t>(off)];
          if (sum == INF) break;
        }
        if (sum < best) { best = sum; best_c = c; }
      }
      nf.tab[static_cast<size_t>(idx)] = best;
      d.arg[static_cast<size_t>(idx)] = best_c;
    }
    for (size_t fi : mine) alive_f[fi] = false;
    gone[v] = true;
    if (scope.empty()) {
      constant += nf.tab[0];
    } else {
      factors.push_back(std::move(nf));
      alive_f.push_back(true);
    }
    decisions.push_back(std::move(d));
  }
  std::vector<int> assign(n, 0);
  for (int k = static_cast<int>(decisions.size()) - 1; k >= 0; --k) {
    const Decision& d = decisions[k];
    long long off = 0;
    for (int u : d.scope) off = off * n_cand[u] + assign[u];
    assign[d.var] = d.arg[static_cast<size_t>(off)];
  }
  for (int i = 0; i < n; ++i) choice_out[i] = assign[i];
  return constant;
}
