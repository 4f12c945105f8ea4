#include "numa.hpp"

#include <cctype>
#include <fstream>
#include <sstream>

namespace hostrt {

static bool read_file(const std::string& path, std::string& out) {
  std::ifstream f(path);
  if (!f) return false;
  std::stringstream ss;
  ss << f.rdbuf();
  out = ss.str();
  return true;
}

static std::string first_line(const std::string& s) {
  const size_t e = s.find('\n');
  return e == std::string::npos ? s : s.substr(0, e);
}

std::vector<int> parse_cpulist(const std::string& text) {
  std::vector<int> out;
  size_t i = 0;
  const size_t n = text.size();
  auto read_int = [&](long& v) {
    while (i < n && std::isspace(static_cast<unsigned char>(text[i]))) ++i;
    if (i >= n || !std::isdigit(static_cast<unsigned char>(text[i]))) return false;
    v = 0;
    while (i < n && std::isdigit(static_cast<unsigned char>(text[i]))) v = v * 10 + (text[i++] - '0');
    return true;
  };
  while (i < n) {
    long a;
    if (!read_int(a)) break;
    long b = a;
    if (i < n && text[i] == '-') {
      ++i;
      if (!read_int(b)) break;
    }
    for (long c = a; c <= b; ++c) out.push_back(static_cast<int>(c));
    while (i < n && (text[i] == ',' || std::isspace(static_cast<unsigned char>(text[i])))) ++i;
  }
  return out;
}

std::vector<int> parse_distances(const std::string& text) {
  std::vector<int> out;
  std::istringstream ss(text);
  int v;
  while (ss >> v) out.push_back(v);
  return out;
}

long parse_meminfo_field(const std::string& text, const std::string& field) {
  // lines look like "Node 0 MemTotal:       65842380 kB"
  size_t pos = text.find(field + ":");
  if (pos == std::string::npos) return -1;
  pos += field.size() + 1;
  while (pos < text.size() && (text[pos] == ' ' || text[pos] == '\t')) ++pos;
  long v = 0;
  bool any = false;
  while (pos < text.size() && std::isdigit(static_cast<unsigned char>(text[pos]))) { v = v * 10 + (text[pos++] - '0'); any = true; }
  return any ? v : -1;
}

NumaInfo::NumaInfo(const std::string& root) {
  std::string online;
  if (!read_file(root + "/online", online)) return;
  const std::vector<int> ids = parse_cpulist(first_line(online));
  if (ids.empty()) return;
  for (int id : ids) {
    NumaNode nd;
    nd.id = id;
    const std::string base = root + "/node" + std::to_string(id);
    std::string s;
    if (!read_file(base + "/cpulist", s)) return;
    nd.cpu_ids = parse_cpulist(first_line(s));
    if (read_file(base + "/distance", s)) nd.distances = parse_distances(first_line(s));
    if (read_file(base + "/meminfo", s)) {
      nd.mem_total_kb = parse_meminfo_field(s, "MemTotal");
      nd.mem_free_kb = parse_meminfo_field(s, "MemFree");
    }
    nodes_.push_back(std::move(nd));
  }
  ok_ = true;
}

int NumaInfo::index_of(int id) const {
  for (size_t i = 0; i < nodes_.size(); ++i) if (nodes_[i].id == id) return static_cast<int>(i);
  return -1;
}
const NumaNode* NumaInfo::node(int id) const {
  const int i = index_of(id);
  return i < 0 ? nullptr : &nodes_[i];
}
const std::vector<int>& NumaInfo::get_node_cpus(int id) const {
  static const std::vector<int> empty;
  const NumaNode* n = node(id);
  return n ? n->cpu_ids : empty;
}
int NumaInfo::distance(int from_id, int to_id) const {
  const NumaNode* f = node(from_id);
  const int ti = index_of(to_id);
  if (!f || ti < 0 || ti >= static_cast<int>(f->distances.size())) return -1;
  return f->distances[ti];
}
int NumaInfo::cpus_per_node() const {
  // the first node that has CPUs: a memory-only node (no cpulist) in front must not report 0 for the machine
  for (const auto& n : nodes_)
    if (!n.cpu_ids.empty()) return static_cast<int>(n.cpu_ids.size());
  return 0;
}
int NumaInfo::cpus_on_node(int id) const { return static_cast<int>(get_node_cpus(id).size()); }
int NumaInfo::total_cpus() const {
  int t = 0;
  for (const auto& n : nodes_) t += static_cast<int>(n.cpu_ids.size());
  return t;
}
std::string NumaInfo::debug_string() const {
  std::ostringstream os;
  os << "NUMA nodes: " << nodes_.size() << "\n";
  for (const auto& n : nodes_) {
    os << "  node " << n.id << ": " << n.cpu_ids.size() << " cpus, " << n.mem_total_kb / 1024 << " MB total, "
       << n.mem_free_kb / 1024 << " MB free, distances [";
    for (size_t i = 0; i < n.distances.size(); ++i) os << (i ? " " : "") << n.distances[i];
    os << "]\n";
  }
  return os.str();
}

}  // namespace hostrt
