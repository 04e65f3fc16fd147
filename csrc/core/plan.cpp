#include "plan.hpp"

#include <sstream>

namespace geeps_b200 {

namespace {

void json_escape(std::ostringstream& o, const std::string& s) {
  o << '"';
  for (char c : s) {
    if (c == '"' || c == '\\') o << '\\' << c;
    else if (c == '\n') o << "\\n";
    else o << c;
  }
  o << '"';
}

const char* op_name(OpType t) {
  switch (t) {
    case OP_READ: return "read";
    case OP_POST_READ: return "post_read";
    case OP_PRE_UPDATE: return "pre_update";
    case OP_UPDATE: return "update";
    case OP_LOCAL_ACCESS: return "local_access";
    case OP_POST_LOCAL_ACCESS: return "post_local_access";
    default: return "clock";
  }
}

}  // namespace

size_t Plan::gpu_rows_total() const {
  size_t param = 0;
  for (auto& kv : tables) param += kv.second.gpu_rows * (1 + (size_t)kv.second.num_oplog_entries);
  return gpu_local_rows + param + staging_rows * (size_t)staging_copies;
}

std::string Plan::to_json() const {
  std::ostringstream o;
  o << "{\"ok\":" << (ok() ? "true" : "false") << ",\"error\":";
  json_escape(o, error);
  o << ",\"warnings\":[";
  for (size_t i = 0; i < warnings.size(); ++i) { if (i) o << ','; json_escape(o, warnings[i]); }
  o << "],\"clock_handle\":" << clock_handle << ",\"capacity_rows\":"
    << (capacity_rows == (size_t)-1 ? -1LL : (long long)capacity_rows)
    << ",\"peak_staging_rows\":" << peak_staging_rows << ",\"staging_rows\":" << staging_rows
    << ",\"staging_copies\":" << staging_copies << ",\"gpu_local_rows\":" << gpu_local_rows
    << ",\"cpu_local_rows\":" << cpu_local_rows << ",\"gpu_param_rows\":" << gpu_param_rows
    << ",\"cpu_param_rows\":" << cpu_param_rows << ",\"uncached_param_rows\":" << uncached_param_rows
    << ",\"max_access_rows\":" << max_access_rows
    << ",\"gpu_rows_total\":" << gpu_rows_total() << ",\"pf_slack\":" << pf_slack << ",\"ops\":[";
  for (size_t i = 0; i < ops.size(); ++i) {
    const OpInfo& p = ops[i];
    if (i) o << ',';
    o << "{\"handle\":" << i << ",\"type\":\"" << op_name(p.type) << "\",\"table\":"
      << (p.local ? -1LL : (long long)p.table) << ",\"num_rows\":" << p.rows.size()
      << ",\"first_row\":" << (p.rows.empty() ? -1LL : (long long)p.rows[0]) << ",\"slack\":" << p.slack
      << ",\"prestep\":" << p.prestep << ",\"post\":" << p.post << ",\"local\":" << (p.local ? 1 : 0)
      << ",\"fetch\":" << (p.fetch ? 1 : 0) << ",\"keep\":" << (p.keep ? 1 : 0) << ",\"one_off\":"
      << (p.one_off ? 1 : 0) << ",\"location\":" << (int)p.location << ",\"direct\":" << (p.direct ? 1 : 0)
      << ",\"needs_staging\":" << (p.needs_staging ? 1 : 0) << ",\"staging_offset\":" << p.staging_offset
      << ",\"store_offset\":" << p.store_offset << ",\"contiguous\":" << (p.contiguous ? 1 : 0)
      << ",\"table_last_write\":" << (p.table_last_write ? 1 : 0) << ",\"num_vals_limit\":" << p.num_vals_limit
      << "}";
  }
  o << "],\"tables\":[";
  bool first = true;
  for (auto& kv : tables) {
    const TablePlan& t = kv.second;
    if (!first) o << ',';
    first = false;
    o << "{\"table_id\":" << t.table_id << ",\"num_rows\":" << t.rows.size() << ",\"gpu_rows\":" << t.gpu_rows
      << ",\"cpu_rows\":" << t.cpu_rows << ",\"pull\":" << (t.pull ? 1 : 0) << ",\"partition_per\":" << t.partition_per
      << ",\"slack\":" << t.slack << ",\"num_oplog_entries\":"
      << t.num_oplog_entries << ",\"shards\":[";
    for (size_t s = 0; s < t.shard_ranges.size(); ++s) {
      if (s) o << ',';
      o << "{\"start\":" << t.shard_ranges[s].start << ",\"stride\":" << t.shard_ranges[s].stride
        << ",\"count\":" << t.shard_ranges[s].count << "}";
    }
    o << "]}";
  }
  o << "]}";
  return o.str();
}

}  // namespace geeps_b200
