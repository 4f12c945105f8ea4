// Stand-alone driver: prints the topology and one PASS/FAIL/SKIP line per scenario, in the order of the
// reference's test executable (test_linux_threading.mojo:555-570).  Exit code = number of failures.
#include "scenarios.hpp"
int main() { return hostrt::run_all_scenarios(true); }
