// PlanCompiler::compile(): see plan.hpp for what is decided here.
#include <algorithm>
#include <set>

#include "plan.hpp"

namespace geeps_b200 {

namespace {
bool is_pre(OpType t) { return t == OP_READ || t == OP_PRE_UPDATE || t == OP_LOCAL_ACCESS; }
bool is_post(OpType t) { return t == OP_POST_READ || t == OP_UPDATE || t == OP_POST_LOCAL_ACCESS; }

struct LocalBatch {
  size_t key = 0;
  size_t rows = 0;
  std::vector<int> pre_ops;
  bool pinned = false;
  size_t offset = 0;
};

size_t peak_of(const std::vector<OpInfo>& ops, const std::vector<char>& staged, size_t* max_access,
               std::vector<char>* in_peak = nullptr) {
  size_t cur = 0, peak = 0, mx = 0;
  std::vector<int> live, best_live;
  for (size_t i = 0; i < ops.size(); ++i) {
    const OpInfo& op = ops[i];
    if (is_pre(op.type) && staged[i]) {
      cur += op.rows.size();
      live.push_back((int)i);
      if (cur > peak) { peak = cur; best_live = live; }
      mx = std::max(mx, op.rows.size());
    } else if (is_post(op.type) && op.prestep >= 0 && staged[op.prestep]) {
      cur -= std::min(cur, ops[op.prestep].rows.size());
      live.erase(std::remove(live.begin(), live.end(), op.prestep), live.end());
    }
  }
  if (max_access) *max_access = mx;
  if (in_peak) {
    in_peak->assign(ops.size(), 0);
    for (int h : best_live) (*in_peak)[h] = 1;
  }
  return peak;
}

size_t colour(std::vector<OpInfo>& ops, const std::vector<char>& staged) {
  struct Live { size_t off, rows; int pre; };
  std::vector<Live> live;
  size_t height = 0;
  for (size_t i = 0; i < ops.size(); ++i) {
    OpInfo& op = ops[i];
    op.needs_staging = false;
    if (is_pre(op.type) && staged[i]) {
      std::sort(live.begin(), live.end(), [](const Live& a, const Live& b) { return a.off < b.off; });
      size_t off = 0;
      for (const Live& l : live) {
        if (off + op.rows.size() <= l.off) break;
        off = std::max(off, l.off + l.rows);
      }
      op.staging_offset = off;
      op.needs_staging = true;
      live.push_back({off, op.rows.size(), (int)i});
      height = std::max(height, off + op.rows.size());
    } else if (is_post(op.type) && op.prestep >= 0 && staged[op.prestep]) {
      for (size_t k = 0; k < live.size(); ++k)
        if (live[k].pre == op.prestep) { live.erase(live.begin() + k); break; }
    }
  }
  return height;
}

// Second strategy: fit every staged access into a pool of exactly `height` rows, taking the lowest free gap
// and the highest free gap in turn.  For a chain of accesses in which only neighbours overlap (a layer's
// input and output) this reaches the peak demand, where first-fit from the bottom fragments.  Offsets are
// committed only if every access fits.
bool colour_two_ended(std::vector<OpInfo>& ops, const std::vector<char>& staged, size_t height) {
  struct Live { size_t off, rows; int pre; };
  std::vector<Live> live;
  std::vector<std::pair<size_t, size_t>> assigned;   // (op index, offset)
  bool low = true;
  for (size_t i = 0; i < ops.size(); ++i) {
    const OpInfo& op = ops[i];
    if (is_pre(op.type) && staged[i]) {
      const size_t need = op.rows.size();
      std::sort(live.begin(), live.end(), [](const Live& a, const Live& b) { return a.off < b.off; });
      bool found = false;
      size_t off = 0, cursor = 0;
      for (size_t k = 0; k <= live.size(); ++k) {
        const size_t gap_end = k < live.size() ? live[k].off : height;
        if (gap_end >= cursor && gap_end - cursor >= need) {
          off = low ? cursor : gap_end - need;
          found = true;
          if (low) break;          // lowest gap wanted: stop at the first; highest gap: keep the last
        }
        if (k < live.size()) cursor = std::max(cursor, live[k].off + live[k].rows);
      }
      if (!found) return false;
      assigned.emplace_back(i, off);
      live.push_back({off, need, (int)i});
      low = !low;
    } else if (is_post(op.type) && op.prestep >= 0 && staged[op.prestep]) {
      for (size_t k = 0; k < live.size(); ++k)
        if (live[k].pre == op.prestep) { live.erase(live.begin() + k); break; }
    }
  }
  for (const auto& a : assigned) { ops[a.first].staging_offset = a.second; ops[a.first].needs_staging = true; }
  return true;
}
}  // namespace

Plan PlanCompiler::compile() const {
  Plan plan;
  plan.ops = ops_;
  std::vector<OpInfo>& ops = plan.ops;
  const size_t n = ops.size();
  const bool gpu = cfg_.device_is_gpu;
  plan.capacity_rows = (!gpu || cfg_.gpu_memory_capacity == (size_t)-1) ? (size_t)-1
                                                                        : cfg_.gpu_memory_capacity / kRowBytes;

  // ---- 1. structure: clock, pre/post links, one-off ops ----
  for (size_t i = 0; i < n; ++i)
    if (ops[i].type == OP_CLOCK) { plan.clock_handle = (int)i; break; }
  if (plan.clock_handle < 0) { plan.error = "the virtual iteration has no Clock"; return plan; }
  for (size_t i = 0; i < n; ++i) {
    OpInfo& op = ops[i];
    op.one_off = (int)i > plan.clock_handle;
    if (is_post(op.type)) {
      const int p = op.prestep;
      const OpType want = op.type == OP_POST_READ ? OP_READ : op.type == OP_UPDATE ? OP_PRE_UPDATE : OP_LOCAL_ACCESS;
      if (p < 0 || p >= (int)i || ops[p].type != want || ops[p].post >= 0) {
        plan.error = "op " + std::to_string(i) + ": bad prestep handle " + std::to_string(p);
        return plan;
      }
      ops[p].post = (int)i;
      op.table = ops[p].table; op.rows = ops[p].rows; op.local = ops[p].local; op.slack = ops[p].slack;
      op.fetch = ops[p].fetch;
    }
    op.num_vals_limit = op.rows.size() * (size_t)kRowFloats;
  }
  for (size_t i = 0; i < n; ++i)
    if (is_pre(ops[i].type) && ops[i].post < 0) {
      plan.error = "op " + std::to_string(i) + " is never released by a post op";
      return plan;
    }

  // ---- 2. tables: row sets, slack, last writes ----
  for (size_t i = 0; i < n; ++i) {
    const OpInfo& op = ops[i];
    if (!is_pre(op.type) || op.local) continue;
    if (op.table >= cfg_.num_tables) { plan.error = "table id " + std::to_string(op.table) + " >= num_tables"; return plan; }
    if (op.rows.empty()) { plan.error = "op " + std::to_string(i) + " has no rows"; return plan; }
    TablePlan& t = plan.tables[op.table];
    t.table_id = op.table;
    for (size_t r : op.rows) t.row_to_idx[r] = 0;
    if (op.type == OP_READ) { t.slack = std::max(t.slack, op.slack); plan.pf_slack = std::max(plan.pf_slack, op.slack); }
    if (op.type == OP_PRE_UPDATE && (int)i < plan.clock_handle) t.written = true;
  }
  for (auto& kv : plan.tables) {
    TablePlan& t = kv.second;
    size_t idx = 0;
    for (auto& rk : t.row_to_idx) { rk.second = idx++; t.rows.push_back(rk.first); }
    if (!t.written) { plan.error = "table " + std::to_string(t.table_id) + " is never updated before the Clock"; return plan; }
    t.num_oplog_entries = cfg_.update_ring ? t.slack + 1 : (cfg_.read_my_writes ? t.slack + 1 : 1);
    const size_t align = t.table_id < cfg_.partition_align.size() ? cfg_.partition_align[t.table_id] : 1;
    Partitioner part(cfg_.partitioner, t.rows.size(), (size_t)cfg_.num_shards, align);
    for (int s = 0; s < cfg_.num_shards; ++s) t.shard_ranges.push_back(part.range_of((size_t)s));
    t.partition_per = part.per();
    t.pull = cfg_.update_ring && t.table_id < cfg_.pull_tables.size() && cfg_.pull_tables[t.table_id];
    if (t.pull) plan.uncached_param_rows += t.rows.size();
    t.location.assign(t.rows.size(), LOC_UNKNOWN);
    t.slot.assign(t.rows.size(), 0);
  }
  {
    std::set<size_t> seen;
    for (int i = plan.clock_handle - 1; i >= 0; --i)
      if (ops[i].type == OP_UPDATE && !ops[i].local && seen.insert(ops[i].table).second) ops[i].table_last_write = true;
  }

  // ---- 3. zero-copy candidates: one ascending run of cache indices, written once per clock ----
  std::map<std::pair<size_t, size_t>, int> write_count;
  for (size_t i = 0; i < n; ++i)
    if (ops[i].type == OP_PRE_UPDATE && !ops[i].local && !ops[i].one_off)
      for (size_t r : ops[i].rows) write_count[{ops[i].table, r}]++;
  std::vector<char> direct_cand(n, 0);
  for (size_t i = 0; i < n; ++i) {
    OpInfo& op = ops[i];
    if (!is_pre(op.type) || op.local) continue;
    const TablePlan& t = plan.tables[op.table];
    bool run = true;
    const size_t first = t.row_to_idx.at(op.rows[0]);
    for (size_t j = 0; j < op.rows.size() && run; ++j) run = t.row_to_idx.at(op.rows[j]) == first + j;
    op.contiguous = run;
    bool once = true;
    if (op.type == OP_PRE_UPDATE)
      for (size_t r : op.rows) once = once && write_count[{op.table, r}] <= 1;
    direct_cand[i] = cfg_.allow_direct && gpu && run && once && !op.one_off;
    // read-my-updates over the update ring: at slack > 0 a read merges the worker's own pending updates into a
    // private copy, so it cannot alias the cache that the shards write in place
    if (op.type == OP_READ && cfg_.read_my_writes && cfg_.update_ring && t.slack > 0) direct_cand[i] = 0;
    // an uncached table has no worker-side copy to alias: its reads land in the staging pool
    if (op.type == OP_READ && t.pull) {
      direct_cand[i] = 0;
      if (!op.one_off && !(run && first == 0 && op.rows.size() == t.rows.size())) {
        plan.error = "read of uncached table " + std::to_string(t.table_id) + " must cover the whole table in ascending row order";
        return plan;
      }
    }
  }

  // ---- 4. worker-local batches: resident in GPU memory, or host memory + staging ----
  std::map<size_t, LocalBatch> batches;
  for (size_t i = 0; i < n; ++i) {
    const OpInfo& op = ops[i];
    if (op.type != OP_LOCAL_ACCESS) continue;
    if (op.rows.empty()) { plan.error = "local access " + std::to_string(i) + " has no rows"; return plan; }
    LocalBatch& b = batches[op.rows[0]];
    if (b.rows && b.rows != op.rows.size()) {
      plan.error = "local batch starting at row " + std::to_string(op.rows[0]) + " is accessed with different sizes";
      return plan;
    }
    b.key = op.rows[0]; b.rows = op.rows.size(); b.pre_ops.push_back((int)i);
  }
  auto staged_for = [&](const std::map<size_t, LocalBatch>& bs) {
    std::vector<char> st(n, 0);
    for (size_t i = 0; i < n; ++i) {
      const OpInfo& op = ops[i];
      if (!is_pre(op.type)) continue;
      if (op.local) st[i] = gpu && !bs.at(op.rows[0]).pinned;
      else st[i] = !direct_cand[i];
    }
    return st;
  };
  auto pinned_rows = [&](const std::map<size_t, LocalBatch>& bs) {
    size_t s = 0;
    for (auto& kv : bs) if (kv.second.pinned) s += kv.second.rows;
    return s;
  };
  // On the NVLINK transport the parameter cache, its update ring and the shard state must be device
  // resident (peers read and write them in place), so they are carved out of the budget first; on the
  // host-staged transport local data comes first and the parameter cache may spill to host memory.
  size_t param_reserved = 0;
  if (cfg_.update_ring)
    for (auto& kv : plan.tables)   // uncached tables keep the update ring resident, but no copy of the rows
      param_reserved += kv.second.rows.size() * ((kv.second.pull ? 0 : 1) + (size_t)kv.second.num_oplog_entries);
  size_t cap = plan.capacity_rows;
  if (gpu && cap != (size_t)-1 && param_reserved) {
    if (param_reserved > cap) {
      plan.error = "GPU memory budget (" + std::to_string(cap) + " rows) is smaller than the device-resident parameter state (" +
                   std::to_string(param_reserved) + " rows)";
      return plan;
    }
    cap -= param_reserved;
  }
  if (gpu) {
    for (auto& kv : batches) kv.second.pinned = true;
    size_t peak = peak_of(ops, staged_for(batches), nullptr);
    if (cap != (size_t)-1 && pinned_rows(batches) + 2 * peak > cap) {
      // not everything fits: start from nothing resident and add batches greedily - first those
      // alive at the staging peak (each one lowers it), then any other that still fits
      for (auto& kv : batches) kv.second.pinned = false;
      bool progress = true;
      while (progress) {
        progress = false;
        std::vector<char> in_peak;
        peak = peak_of(ops, staged_for(batches), nullptr, &in_peak);
        LocalBatch* best = nullptr;
        bool best_in_peak = false;
        for (auto& kv : batches) {
          LocalBatch& b = kv.second;
          if (b.pinned) continue;
          b.pinned = true;
          const size_t new_peak = peak_of(ops, staged_for(batches), nullptr);
          const bool fits = pinned_rows(batches) + 2 * new_peak <= cap;
          b.pinned = false;
          if (!fits) continue;
          bool inpk = false;
          for (int h : b.pre_ops) inpk = inpk || in_peak[h];
          if (!best || (inpk && !best_in_peak) || (inpk == best_in_peak && b.rows > best->rows)) {
            best = &b; best_in_peak = inpk;
          }
        }
        if (best) { best->pinned = true; progress = true; }
      }
    }
  }
  {
    size_t goff = 0, coff = 0;
    for (auto& kv : batches) {
      LocalBatch& b = kv.second;
      if (!gpu || !b.pinned) { b.offset = coff; coff += b.rows; }
      else { b.offset = goff; goff += b.rows; }
    }
    plan.gpu_local_rows = goff;
    plan.cpu_local_rows = coff;
    if (gpu && coff > 0) {
      const std::string msg = std::to_string(coff) + " rows of worker-local data do not fit in GPU memory and are swapped from host memory";
      if (cfg_.mm_warning_level >= 2) { plan.error = msg; return plan; }
      plan.warnings.push_back(msg);
    }
  }
  std::vector<char> staged = staged_for(batches);
  plan.peak_staging_rows = peak_of(ops, staged, &plan.max_access_rows);

  // ---- 5. parameter cache: GPU while it fits (first fit in op order), host memory after that ----
  size_t avail = (size_t)-1;
  if (gpu && cap != (size_t)-1 && !param_reserved) {
    const size_t taken = plan.gpu_local_rows + 2 * plan.peak_staging_rows;
    avail = cap > taken ? cap - taken : 0;
  }
  size_t used_param = 0;  // rows incl. oplog copies
  for (size_t i = 0; i < n; ++i) {
    const OpInfo& op = ops[i];
    if (!is_pre(op.type) || op.local) continue;
    TablePlan& t = plan.tables[op.table];
    size_t fresh = 0;
    for (size_t r : op.rows) if (t.location[t.row_to_idx[r]] == LOC_UNKNOWN) ++fresh;
    if (!fresh) continue;
    const size_t need = fresh * (1 + (size_t)t.num_oplog_entries);
    const int loc = !gpu ? LOC_CPU : (avail == (size_t)-1 || used_param + need <= avail) ? LOC_GPU : LOC_CPU;
    if (loc == LOC_GPU) used_param += need;
    for (size_t r : op.rows) {
      const size_t idx = t.row_to_idx[r];
      if (t.location[idx] == LOC_UNKNOWN) t.location[idx] = loc;
    }
  }
  for (auto& kv : plan.tables) {
    TablePlan& t = kv.second;
    for (size_t idx = 0; idx < t.rows.size(); ++idx) {
      if (t.location[idx] == LOC_GPU) t.slot[idx] = t.gpu_rows++;
      else t.slot[idx] = t.cpu_rows++;
    }
    plan.gpu_param_rows += t.gpu_rows;
    plan.cpu_param_rows += t.cpu_rows;
  }
  if (gpu && plan.cpu_param_rows > 0) {
    const std::string msg = std::to_string(plan.cpu_param_rows) + " parameter rows do not fit in the GPU parameter cache and are cached in host memory";
    if (cfg_.mm_warning_level >= 3) { plan.error = msg; return plan; }
    plan.warnings.push_back(msg);
  }

  // ---- 6. per-op placement, gather indices, final staging layout ----
  for (size_t i = 0; i < n; ++i) {
    OpInfo& op = ops[i];
    if (!is_pre(op.type)) continue;
    if (op.local) {
      const LocalBatch& b = batches[op.rows[0]];
      op.location = (gpu && b.pinned) ? LOC_GPU : LOC_CPU;
      op.store_offset = b.offset;
      op.direct = !staged[i];
      continue;
    }
    TablePlan& t = plan.tables[op.table];
    const int loc0 = t.location[t.row_to_idx[op.rows[0]]];
    bool same = true, slot_run = true;
    op.index.clear();
    for (size_t j = 0; j < op.rows.size(); ++j) {
      const size_t idx = t.row_to_idx[op.rows[j]];
      same = same && t.location[idx] == loc0;
      slot_run = slot_run && t.slot[idx] == t.slot[t.row_to_idx[op.rows[0]]] + j;
      op.index.push_back(DoubleIndex((int64_t)j, (int64_t)t.slot[idx]));
    }
    if (!same) {
      plan.error = "row batch of op " + std::to_string(i) + " straddles the GPU and host parameter caches";
      return plan;
    }
    op.location = (DataLocation)loc0;
    op.store_offset = t.slot[t.row_to_idx[op.rows[0]]];
    op.contiguous = op.contiguous && slot_run;
    op.direct = direct_cand[i] && loc0 == LOC_GPU && slot_run;
    staged[i] = !op.direct;
  }
  for (size_t i = 0; i < n; ++i)
    if (is_post(ops[i].type)) {
      const OpInfo& pre = ops[ops[i].prestep];
      ops[i].location = pre.location; ops[i].direct = pre.direct; ops[i].store_offset = pre.store_offset;
      ops[i].contiguous = pre.contiguous;
    }
  {
    std::map<size_t, int> last_post;
    for (size_t i = 0; i < n; ++i)
      if (ops[i].type == OP_POST_LOCAL_ACCESS && !ops[i].one_off) last_post[ops[i].rows[0]] = (int)i;
    for (auto& kv : last_post) ops[kv.second].last_access_of_batch = true;
  }
  plan.peak_staging_rows = peak_of(ops, staged, &plan.max_access_rows);
  plan.staging_rows = colour(ops, staged);
  if (plan.staging_rows > plan.peak_staging_rows && colour_two_ended(ops, staged, plan.peak_staging_rows))
    plan.staging_rows = plan.peak_staging_rows;
  for (size_t i = 0; i < n; ++i)
    if (is_post(ops[i].type)) {
      ops[i].needs_staging = ops[ops[i].prestep].needs_staging;
      ops[i].staging_offset = ops[ops[i].prestep].staging_offset;
    }
  plan.staging_copies = 2;
  if (gpu && cap != (size_t)-1) {
    const size_t fixed = plan.gpu_local_rows + (param_reserved ? 0 : used_param);   // reserved rows already left `cap`
    if (fixed + 2 * plan.staging_rows > cap) {
      const std::string msg = "staging pool cannot be double buffered: need " + std::to_string(2 * plan.staging_rows) +
                              " rows, " + std::to_string(cap > fixed ? cap - fixed : 0) + " left";
      if (cfg_.mm_warning_level >= 1) { plan.error = msg; return plan; }
      plan.warnings.push_back(msg);
      plan.staging_copies = 1;
      if (fixed + plan.staging_rows > cap) { plan.error = "GPU memory budget too small even for single-buffered staging"; return plan; }
    }
  }
  return plan;
}

}  // namespace geeps_b200
