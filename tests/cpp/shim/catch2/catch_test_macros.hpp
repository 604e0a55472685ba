// Minimal stand-in for the parts of Catch2 v3 that Fusilli's samples and tests use
// (TEST_CASE, SECTION, REQUIRE, REQUIRE_FALSE, CHECK, INFO, FAIL, GENERATE over a value list,
// REQUIRE_THAT with ContainsSubstring). Catch2 itself is not installed on this machine.
// One translation unit per executable; main() is provided here.
#pragma once

#include <cstdio>
#include <cstdlib>
#include <functional>
#include <iostream>
#include <sstream>
#include <string>
#include <vector>

namespace catch_shim {

struct TestCase {
  const char *name;
  void (*fn)();
};
inline std::vector<TestCase> &registry() {
  static std::vector<TestCase> r;
  return r;
}
struct Registrar {
  Registrar(const char *name, void (*fn)()) { registry().push_back({name, fn}); }
};

// GENERATE: every site is a digit of an odometer; the test case re-runs until all
// combinations of all sites have been visited.
struct GenState {
  struct Site { int id; size_t index, count; };
  std::vector<Site> sites;
  size_t cursor = 0; // position of the next GENERATE call within the current run
};
inline GenState &gen() {
  static GenState g;
  return g;
}
template <typename T> T generate(int id, std::vector<T> values) {
  GenState &g = gen();
  if (g.cursor == g.sites.size()) g.sites.push_back({id, 0, values.size()});
  GenState::Site &s = g.sites[g.cursor++];
  s.count = values.size();
  return values[s.index];
}
// advances the odometer; false when every combination has been run
inline bool next_combination() {
  GenState &g = gen();
  for (size_t i = g.sites.size(); i > 0; --i) {
    if (++g.sites[i - 1].index < g.sites[i - 1].count) {
      g.sites.resize(i);
      return true;
    }
  }
  return false;
}

inline int &failures() {
  static int f = 0;
  return f;
}
inline std::string &info_line() {
  static std::string s;
  return s;
}
struct AbortTest {};
inline void fail(const char *expr, const char *file, int line, const std::string &extra = "") {
  ++failures();
  std::cerr << file << ":" << line << ": FAILED: " << expr;
  if (!extra.empty()) std::cerr << " (" << extra << ")";
  if (!info_line().empty()) std::cerr << " [" << info_line() << "]";
  std::cerr << std::endl;
  throw AbortTest{};
}

// SECTION: each run of a test case enters, at every nesting level, the first section that is not
// finished yet and skips its later siblings; the case re-runs until no section was skipped, so every
// leaf section sees a fresh execution of the code around it (as in Catch2).
struct SectionNode {
  std::string key;
  std::vector<SectionNode> children;
  bool done = false, entered_child = false, rerun = false;
  SectionNode *child(const std::string &k) {
    for (auto &c : children)
      if (c.key == k) return &c;
    children.reserve(64); // pointers into the vector stay valid for any realistic test
    children.push_back(SectionNode{k});
    return &children.back();
  }
};
inline SectionNode &section_root() {
  static SectionNode r;
  return r;
}
inline SectionNode *&section_current() {
  static SectionNode *c = &section_root();
  return c;
}
struct SectionGuard {
  SectionNode *parent = nullptr, *self = nullptr;
  explicit SectionGuard(const std::string &key) {
    SectionNode *cur = section_current();
    SectionNode *c = cur->child(key);
    if (c->done) return;
    if (cur->entered_child) {
      cur->rerun = true;
      return;
    }
    cur->entered_child = true;
    parent = cur;
    self = c;
    self->entered_child = false;
    self->rerun = false;
    section_current() = self;
  }
  ~SectionGuard() {
    if (!self) return;
    if (!self->rerun) self->done = true;
    else parent->rerun = true;
    section_current() = parent;
  }
  explicit operator bool() const { return self != nullptr; }
};

inline int run_all() {
  int ran = 0;
  for (const TestCase &tc : registry()) {
    gen().sites.clear();
    do {
      section_root() = SectionNode{};
      int guard = 0;
      do {
        section_root().entered_child = false;
        section_root().rerun = false;
        section_current() = &section_root();
        gen().cursor = 0;
        info_line().clear();
        try {
          tc.fn();
        } catch (const AbortTest &) {
        }
        ++ran;
      } while (section_root().rerun && ++guard < 1000);
    } while (next_combination());
    std::cout << (failures() ? "[FAIL] " : "[ ok ] ") << tc.name << std::endl;
  }
  std::cout << ran << " run(s), " << failures() << " failure(s)" << std::endl;
  return failures() ? 1 : 0;
}

} // namespace catch_shim

namespace Catch {
template <typename T> struct StringMaker {
  static std::string convert(const T &) { return "?"; }
};
namespace Matchers {
struct ContainsSubstring {
  std::string needle;
  explicit ContainsSubstring(std::string n) : needle(std::move(n)) {}
  bool match(const std::string &s) const { return s.find(needle) != std::string::npos; }
};
} // namespace Matchers
} // namespace Catch

#define CATCH_SHIM_CAT2(a, b) a##b
#define CATCH_SHIM_CAT(a, b) CATCH_SHIM_CAT2(a, b)
#define TEST_CASE(...) CATCH_SHIM_TEST_CASE(CATCH_SHIM_CAT(catch_shim_test_, __COUNTER__), __VA_ARGS__)
#define CATCH_SHIM_TEST_CASE(fn, name, ...)                                                          \
  static void fn();                                                                                  \
  static catch_shim::Registrar CATCH_SHIM_CAT(fn, _reg)(name, &fn);                                  \
  static void fn()
#define SECTION(...)                                                                                 \
  if (catch_shim::SectionGuard CATCH_SHIM_CAT(catch_shim_section_, __LINE__) =                       \
          catch_shim::SectionGuard(std::string(__FILE__) + ":" + std::to_string(__LINE__)))
#define REQUIRE(...)                                                                                 \
  do {                                                                                               \
    if (!(__VA_ARGS__)) catch_shim::fail(#__VA_ARGS__, __FILE__, __LINE__);                          \
  } while (false)
#define CHECK(...) REQUIRE(__VA_ARGS__)
#define REQUIRE_FALSE(...)                                                                           \
  do {                                                                                               \
    if ((__VA_ARGS__)) catch_shim::fail("!(" #__VA_ARGS__ ")", __FILE__, __LINE__);                  \
  } while (false)
#define REQUIRE_THAT(value, matcher)                                                                 \
  do {                                                                                               \
    if (!(matcher).match(value)) catch_shim::fail(#value " " #matcher, __FILE__, __LINE__);          \
  } while (false)
#define INFO(msg)                                                                                    \
  do {                                                                                               \
    std::ostringstream catch_shim_os;                                                                \
    catch_shim_os << msg;                                                                            \
    catch_shim::info_line() = catch_shim_os.str();                                                   \
  } while (false)
#define FAIL(msg)                                                                                    \
  do {                                                                                               \
    std::ostringstream catch_shim_os;                                                                \
    catch_shim_os << msg;                                                                            \
    catch_shim::fail("FAIL", __FILE__, __LINE__, catch_shim_os.str());                               \
  } while (false)
namespace catch_shim {
template <typename T, typename... R> inline std::vector<std::decay_t<T>> values(T &&first, R &&...rest) {
  std::vector<std::decay_t<T>> v;
  v.emplace_back(std::forward<T>(first));
  (v.emplace_back(std::forward<R>(rest)), ...);
  return v;
}
} // namespace catch_shim
// Arguments may hold braced lists with commas, so they are only ever passed on whole.
#define GENERATE(...) catch_shim::generate(__COUNTER__, catch_shim::values(__VA_ARGS__))

// A second translation unit of the same program (a shared helper) is compiled with
// -DCATCH_SHIM_NO_MAIN; the registry and counters above are inline and therefore shared.
#ifndef CATCH_SHIM_NO_MAIN
int main() { return catch_shim::run_all(); }
#endif
