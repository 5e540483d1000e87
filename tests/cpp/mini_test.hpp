// A very small test harness (the image has no GoogleTest): TEST(Suite, Name) { ... } registers a case,
// EXPECT_* record failures and continue, ASSERT_* record and leave the case, SKIP_TEST(msg) leaves it
// as skipped. main() runs every case (optionally filtered by a substring) and returns 1 on failure.
#pragma once

#include <cmath>
#include <cstdio>
#include <cstring>
#include <functional>
#include <sstream>
#include <string>
#include <type_traits>
#include <vector>

namespace mini {

struct Case {
    std::string name;
    std::function<void()> body;
};
inline std::vector<Case>& Cases() {
    static std::vector<Case> cases;
    return cases;
}
struct State {
    int failures = 0;
    bool skipped = false;
    std::string skip_reason;
};
inline State& Current() {
    static State s;
    return s;
}
struct Registrar {
    Registrar(const char* suite, const char* name, std::function<void()> body) {
        Cases().push_back({std::string(suite) + "." + name, std::move(body)});
    }
};
inline void Fail(const char* file, int line, const std::string& what) {
    ++Current().failures;
    std::printf("  FAILED %s:%d: %s\n", file, line, what.c_str());
}
template <typename T>
void Put(std::ostringstream& os, const T& v) {
    if constexpr (std::is_enum_v<T>) os << static_cast<long long>(v);
    else os << v;
}
template <typename A, typename B>
std::string Show(const A& a, const B& b) {
    std::ostringstream os;
    os << "left=";
    Put(os, a);
    os << " right=";
    Put(os, b);
    return os.str();
}
inline int RunAll(int argc, char** argv) {
    const char* filter = argc > 1 ? argv[1] : "";
    int failed = 0, passed = 0, skipped = 0;
    for (const Case& c : Cases()) {
        if (filter[0] != '\0' && c.name.find(filter) == std::string::npos) continue;
        Current() = State{};
        std::printf("[ RUN  ] %s\n", c.name.c_str());
        c.body();
        if (Current().skipped) {
            ++skipped;
            std::printf("[ SKIP ] %s (%s)\n", c.name.c_str(), Current().skip_reason.c_str());
        } else if (Current().failures > 0) {
            ++failed;
            std::printf("[ FAIL ] %s\n", c.name.c_str());
        } else {
            ++passed;
            std::printf("[  OK  ] %s\n", c.name.c_str());
        }
        std::fflush(stdout);
    }
    std::printf("SUMMARY passed=%d failed=%d skipped=%d\n", passed, failed, skipped);
    return failed == 0 ? 0 : 1;
}

}  // namespace mini

#define TEST(suite, name)                                                         \
    static void suite##_##name##_body();                                          \
    static mini::Registrar suite##_##name##_reg(#suite, #name, suite##_##name##_body); \
    static void suite##_##name##_body()

#define MINI_CHECK(cond, text, fatal)                       \
    do {                                                    \
        if (!(cond)) {                                      \
            mini::Fail(__FILE__, __LINE__, text);           \
            if (fatal) return;                              \
        }                                                   \
    } while (0)

#define EXPECT_TRUE(x) MINI_CHECK((x), std::string("expected true: ") + #x, false)
#define EXPECT_FALSE(x) MINI_CHECK(!(x), std::string("expected false: ") + #x, false)
#define ASSERT_TRUE(x) MINI_CHECK((x), std::string("expected true: ") + #x, true)
#define ASSERT_FALSE(x) MINI_CHECK(!(x), std::string("expected false: ") + #x, true)
#define EXPECT_EQ(a, b) MINI_CHECK((a) == (b), std::string(#a " == " #b ": ") + mini::Show((a), (b)), false)
#define ASSERT_EQ(a, b) MINI_CHECK((a) == (b), std::string(#a " == " #b ": ") + mini::Show((a), (b)), true)
#define EXPECT_NE(a, b) MINI_CHECK((a) != (b), std::string(#a " != " #b), false)
#define EXPECT_LT(a, b) MINI_CHECK((a) < (b), std::string(#a " < " #b ": ") + mini::Show((a), (b)), false)
#define EXPECT_LE(a, b) MINI_CHECK((a) <= (b), std::string(#a " <= " #b ": ") + mini::Show((a), (b)), false)
#define EXPECT_GT(a, b) MINI_CHECK((a) > (b), std::string(#a " > " #b ": ") + mini::Show((a), (b)), false)
#define EXPECT_GE(a, b) MINI_CHECK((a) >= (b), std::string(#a " >= " #b ": ") + mini::Show((a), (b)), false)
#define EXPECT_NEAR(a, b, tol) MINI_CHECK(std::fabs(double(a) - double(b)) <= (tol), std::string(#a " ~ " #b ": ") + mini::Show((a), (b)), false)
#define EXPECT_STREQ(a, b) MINI_CHECK(std::strcmp((a), (b)) == 0, std::string(#a " == " #b ": ") + mini::Show((a), (b)), false)
#define EXPECT_HAS(text, part) MINI_CHECK(std::string(text).find(part) != std::string::npos, std::string("\"") + std::string(text) + "\" lacks \"" + (part) + "\"", false)
#define SKIP_TEST(reason)                      \
    do {                                       \
        mini::Current().skipped = true;        \
        mini::Current().skip_reason = reason;  \
        return;                                \
    } while (0)
