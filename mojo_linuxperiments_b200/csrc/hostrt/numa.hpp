// NUMA topology from sysfs: online nodes, CPUs per node, distance matrix, MemTotal / MemFree.
// Capability parity: numa/numa.mojo:6-176 of the reference (NumaInfo, NumaNode, get_current_cpu_and_node).
// Differences by design: nodes are looked up by their id (sparse ids work), the sysfs root is a parameter so
// tests can point it at a fixture tree, and a failed read yields an empty topology with ok() == false.
#pragma once
#include <string>
#include <vector>

#include "cpumask.hpp"
#include "sys.hpp"

namespace hostrt {

struct NumaNode {
  int id = -1;
  std::vector<int> cpu_ids;
  std::vector<int> distances;       // indexed by position in NumaInfo::nodes()
  long mem_total_kb = 0;
  long mem_free_kb = 0;
};

std::vector<int> parse_cpulist(const std::string& text);      // "0-3,8,10-11" -> {0,1,2,3,8,10,11}
std::vector<int> parse_distances(const std::string& text);    // "10 21 21" -> {10,21,21}
long parse_meminfo_field(const std::string& text, const std::string& field);   // value in kB, -1 if absent

class NumaInfo {
 public:
  explicit NumaInfo(const std::string& sysfs_root = "/sys/devices/system/node");
  bool ok() const { return ok_; }
  int num_nodes() const { return static_cast<int>(nodes_.size()); }
  const std::vector<NumaNode>& nodes() const { return nodes_; }
  const NumaNode* node(int id) const;                 // by node id; nullptr if unknown
  int index_of(int id) const;                         // position in nodes(), -1 if unknown
  const std::vector<int>& get_node_cpus(int id) const;
  template <size_t Bytes = 128>
  CpuMask<Bytes> get_node_mask(int id) const {
    CpuMask<Bytes> m;
    for (int c : get_node_cpus(id)) m.set(c);
    return m;
  }
  int distance(int from_id, int to_id) const;         // -1 for an unknown node
  int cpus_per_node() const;                          // count on the first node (uniform machines)
  int cpus_on_node(int id) const;
  int total_cpus() const;
  std::string debug_string() const;

 private:
  std::vector<NumaNode> nodes_;
  bool ok_ = false;
};

struct CpuNode { int cpu; int node; };
inline CpuNode get_current_cpu_and_node() {            // one getcpu syscall
  unsigned c = 0, n = 0;
  sys_getcpu(&c, &n);
  return {static_cast<int>(c), static_cast<int>(n)};
}

}  // namespace hostrt
