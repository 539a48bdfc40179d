// Minimal unit-test framework for the C++ layer: TEST(suite, name) { EXPECT_*/ASSERT_* }, one process or several
// (MSCCLPP_TEST_RANK / MSCCLPP_TEST_NRANKS from the environment), a perf-result line format, exit code = failures.
// The reference has a framework of the same shape built on MPI (test/framework.hpp:22-69); this one gets its ranks
// from the environment so that a plain launcher (fork, torchrun, pytest) can start them.
#pragma once

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <functional>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

namespace testing {

struct TestCase {
  std::string suite, name;
  std::function<void()> body;
};

inline std::vector<TestCase>& registry() {
  static std::vector<TestCase> r;
  return r;
}
inline int& failures() {
  static int f = 0;
  return f;
}
inline int rank() {
  const char* r = std::getenv("MSCCLPP_TEST_RANK");
  return r ? std::atoi(r) : 0;
}
inline int nRanks() {
  const char* r = std::getenv("MSCCLPP_TEST_NRANKS");
  return r ? std::atoi(r) : 1;
}

struct Registrar {
  Registrar(const char* suite, const char* name, std::function<void()> body) { registry().push_back({suite, name, std::move(body)}); }
};

struct AssertionFailure : std::runtime_error {
  using std::runtime_error::runtime_error;
};

inline void reportFailure(const char* file, int line, const std::string& what, bool fatal) {
  std::fprintf(stderr, "[rank %d] %s:%d: %s\n", rank(), file, line, what.c_str());
  failures()++;
  if (fatal) throw AssertionFailure(what);
}

// One line per measurement, easy to grep and to parse: PERF <name> <value> <unit> key=value ...
inline void reportPerf(const std::string& name, double value, const std::string& unit, const std::string& extra = "") {
  if (rank() == 0) std::printf("PERF %s %.4f %s %s\n", name.c_str(), value, unit.c_str(), extra.c_str());
}

struct Timer {
  std::chrono::steady_clock::time_point t0 = std::chrono::steady_clock::now();
  double elapsedUs() const { return std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count(); }
};

inline int runAll(int argc, char** argv) {
  std::string filter = argc > 1 ? argv[1] : "";
  int ran = 0;
  for (auto& t : registry()) {
    const std::string full = t.suite + "." + t.name;
    if (!filter.empty() && full.find(filter) == std::string::npos) continue;
    const int before = failures();
    if (rank() == 0) std::printf("[ RUN      ] %s\n", full.c_str());
    try {
      t.body();
    } catch (const AssertionFailure&) {
    } catch (const std::exception& e) {
      reportFailure(__FILE__, __LINE__, std::string("uncaught exception: ") + e.what(), false);
    }
    if (rank() == 0) std::printf("[ %s ] %s\n", failures() == before ? "      OK" : "  FAILED", full.c_str());
    ran++;
  }
  if (rank() == 0) std::printf("%d tests, %d failures\n", ran, failures());
  return failures() == 0 ? 0 : 1;
}

}  // namespace testing

#define TEST(suite, name)                                                            \
  static void suite##_##name##_body();                                               \
  static ::testing::Registrar suite##_##name##_registrar(#suite, #name, suite##_##name##_body); \
  static void suite##_##name##_body()

#define MSCCLPP_TEST_STR(x) ([&] { std::ostringstream os_; os_ << (x); return os_.str(); }())
#define EXPECT_TRUE(c) do { if (!(c)) ::testing::reportFailure(__FILE__, __LINE__, "expected true: " #c, false); } while (0)
#define ASSERT_TRUE(c) do { if (!(c)) ::testing::reportFailure(__FILE__, __LINE__, "expected true: " #c, true); } while (0)
#define EXPECT_EQ(a, b) do { auto a_ = (a); auto b_ = (b); if (!(a_ == b_)) ::testing::reportFailure(__FILE__, __LINE__, std::string(#a " == " #b ": ") + MSCCLPP_TEST_STR(a_) + " vs " + MSCCLPP_TEST_STR(b_), false); } while (0)
#define ASSERT_EQ(a, b) do { auto a_ = (a); auto b_ = (b); if (!(a_ == b_)) ::testing::reportFailure(__FILE__, __LINE__, std::string(#a " == " #b ": ") + MSCCLPP_TEST_STR(a_) + " vs " + MSCCLPP_TEST_STR(b_), true); } while (0)
#define EXPECT_THROW(stmt, type) do { bool thrown_ = false; try { stmt; } catch (const type&) { thrown_ = true; } catch (...) {} if (!thrown_) ::testing::reportFailure(__FILE__, __LINE__, "expected " #type " from: " #stmt, false); } while (0)
