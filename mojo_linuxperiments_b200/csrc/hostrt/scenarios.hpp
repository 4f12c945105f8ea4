#pragma once
#include <cstddef>

namespace hostrt {
enum ScenarioResult : int { SC_PASS = 0, SC_FAIL = 1, SC_SKIP = 2 };
int scenario_count();
const char* scenario_name(int i);
int scenario_run(int i, char* detail, size_t n);
// runs every scenario in the reference's order; returns the number of failures
int run_all_scenarios(bool print);
}  // namespace hostrt
