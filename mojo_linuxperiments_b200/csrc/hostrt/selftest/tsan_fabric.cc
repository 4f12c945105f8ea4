// Thread-sanitizer run of the collective protocols of the host fabric (built with -fsanitize=thread and
// -DHOSTRT_STD_THREADS, so the ranks are std::threads the sanitizer can see): the epoch all-reduce over persistent
// workers, and the token exchange with its flag / buffer-parity / acknowledgement protocol, in every mode.
// Exit code 0: the protocols ran, produced the right values and the sanitizer reported no race (a report makes the
// process exit with TSAN_OPTIONS' exitcode, 66 by default).
#include <cmath>
#include <cstdio>
#include <vector>

#include "collectives.hpp"
#include "numa.hpp"

int main() {
  using namespace hostrt;
  NumaInfo info;
  int failures = 0;
  for (int world : {2, 4}) {
    std::vector<double> in(world), out(world, 0.0);
    double want = 0;
    for (int r = 0; r < world; ++r) { in[r] = 0.5 + r; want += in[r]; }
    // every round all-reduces the previous round's result again: sum * world^(rounds - 1)
    const int rounds = 12;
    const long st = fabric_allreduce(info, world, in.data(), out.data(), rounds, 5'000'000'000l, -1);
    want *= std::pow(static_cast<double>(world), rounds - 1);
    bool ok = st == 0;
    for (int r = 0; r < world; ++r) ok = ok && std::fabs(out[r] - want) < 1e-9 * want && out[r] == out[0];
    std::printf("[%s] fabric_allreduce world %d status %ld\n", ok ? "PASS" : "FAIL", world, st);
    failures += !ok;
    for (int mode = 1; mode <= 3; ++mode) {
      int mism = -1;
      const long se = fabric_token_exchange(info, world, 8, 4, 60, 5'000'000'000l, 7u, mode, 0, &mism);
      const bool eok = se == 0 && mism == 0;
      std::printf("[%s] fabric_token_exchange world %d mode %d status %ld mismatches %d\n", eok ? "PASS" : "FAIL", world, mode, se, mism);
      failures += !eok;
    }
  }
  return failures;
}
