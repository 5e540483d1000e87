// A small stand-in for <gtest/gtest.h> (GoogleTest is not installed where these tests are built).
//
// It implements the part of the GoogleTest interface that the reference's own test sources use, so that
// those files compile UNMODIFIED: TEST(), EXPECT_* / ASSERT_* with `<< message` streaming, GTEST_SKIP(),
// ADD_FAILURE(), ::testing::Test::HasFatalFailure(), and a main() (when GTEST_SHIM_MAIN is defined) that
// understands --gtest_filter=POSITIVE[-NEGATIVE] with ':'-separated '*' patterns. Output follows
// GoogleTest's line format closely enough for the same log scrapers.
#pragma once

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <functional>
#include <sstream>
#include <string>
#include <type_traits>
#include <utility>
#include <vector>

namespace testing {

namespace internal {

template <typename T, typename = void>
struct IsStreamable : std::false_type {};
template <typename T>
struct IsStreamable<T, std::void_t<decltype(std::declval<std::ostream&>() << std::declval<const T&>())>> : std::true_type {};

template <typename T>
void PrintValue(std::ostream& os, const T& value) {
    if constexpr (std::is_same_v<T, bool>) {
        os << (value ? "true" : "false");
    } else if constexpr (std::is_null_pointer_v<T>) {
        os << "nullptr";
    } else if constexpr (std::is_enum_v<T>) {
        os << static_cast<long long>(value);
    } else if constexpr (std::is_same_v<T, signed char> || std::is_same_v<T, unsigned char>) {
        os << static_cast<int>(value);
    } else if constexpr (IsStreamable<T>::value) {
        os << value;
    } else {
        os << "<" << sizeof(T) << "-byte object>";
    }
}

struct CaseState {
    int failures = 0;
    bool fatal = false;
    bool skipped = false;
    std::string skip_text;
};
inline CaseState& State() {
    static CaseState state;
    return state;
}

struct Case {
    std::string name;
    std::function<void()> body;
};
inline std::vector<Case>& Cases() {
    static std::vector<Case> cases;
    return cases;
}
struct Registrar {
    Registrar(const char* suite, const char* name, std::function<void()> body) {
        Cases().push_back({std::string(suite) + "." + name, std::move(body)});
    }
};

}  // namespace internal

class Message {
public:
    Message() = default;
    template <typename T>
    Message& operator<<(const T& value) {
        internal::PrintValue(text_, value);
        return *this;
    }
    Message& operator<<(const char* value) {
        text_ << (value != nullptr ? value : "(null)");
        return *this;
    }
    std::string str() const { return text_.str(); }

private:
    std::ostringstream text_;
};

class AssertionResult {
public:
    explicit AssertionResult(bool ok, std::string text = std::string()) : ok_(ok), text_(std::move(text)) {}
    explicit operator bool() const { return ok_; }
    const std::string& text() const { return text_; }

private:
    bool ok_;
    std::string text_;
};

class Test {
public:
    static bool HasFatalFailure() { return internal::State().fatal; }
    static bool HasFailure() { return internal::State().failures > 0; }
    static bool IsSkipped() { return internal::State().skipped; }
};

namespace internal {

// `Reporter(...) = Message() << ...` records one failure; operator= has lower precedence than <<, which is what
// lets the macros below accept a trailing `<< text`.
class Reporter {
public:
    Reporter(const char* file, int line, bool fatal, std::string what)
        : file_(file), line_(line), fatal_(fatal), what_(std::move(what)) {}
    void operator=(const Message& message) const {
        CaseState& s = State();
        ++s.failures;
        if (fatal_) s.fatal = true;
        const std::string extra = message.str();
        std::printf("%s:%d: Failure\n%s%s%s\n", file_, line_, what_.c_str(), extra.empty() ? "" : "\n", extra.c_str());
        std::fflush(stdout);
    }

private:
    const char* file_;
    int line_;
    bool fatal_;
    std::string what_;
};

class Skipper {
public:
    void operator=(const Message& message) const {
        State().skipped = true;
        State().skip_text = message.str();
    }
};

template <typename A, typename B>
std::string Sides(const char* a_text, const char* b_text, const A& a, const B& b, const char* relation) {
    std::ostringstream os;
    os << "Expected: (" << a_text << ") " << relation << " (" << b_text << "), actual: ";
    PrintValue(os, a);
    os << " vs ";
    PrintValue(os, b);
    return os.str();
}

#define GTEST_SHIM_COMPARE(Name, op)                                                                 \
    template <typename A, typename B>                                                                \
    AssertionResult Cmp##Name(const char* a_text, const char* b_text, const A& a, const B& b) {     \
        if (a op b) return AssertionResult(true);                                                    \
        return AssertionResult(false, Sides(a_text, b_text, a, b, #op));                             \
    }
GTEST_SHIM_COMPARE(EQ, ==)
GTEST_SHIM_COMPARE(NE, !=)
GTEST_SHIM_COMPARE(LT, <)
GTEST_SHIM_COMPARE(LE, <=)
GTEST_SHIM_COMPARE(GT, >)
GTEST_SHIM_COMPARE(GE, >=)
#undef GTEST_SHIM_COMPARE

inline AssertionResult CmpStrEq(const char* a_text, const char* b_text, const char* a, const char* b) {
    const bool same = (a == nullptr || b == nullptr) ? a == b : std::strcmp(a, b) == 0;
    if (same) return AssertionResult(true);
    return AssertionResult(false, Sides(a_text, b_text, std::string(a ? a : "(null)"), std::string(b ? b : "(null)"), "=="));
}
inline AssertionResult CmpNear(const char* a_text, const char* b_text, double a, double b, double tolerance) {
    if (std::fabs(a - b) <= tolerance) return AssertionResult(true);
    std::ostringstream os;
    os << "The difference between " << a_text << " and " << b_text << " is " << std::fabs(a - b) << ", which exceeds "
       << tolerance << " (" << a << " vs " << b << ")";
    return AssertionResult(false, os.str());
}
// 4-ULP comparison, as GoogleTest's EXPECT_FLOAT_EQ
inline AssertionResult CmpFloatEq(const char* a_text, const char* b_text, float a, float b) {
    auto biased = [](float f) {
        uint32_t bits;
        std::memcpy(&bits, &f, sizeof(bits));
        return (bits & 0x80000000u) ? ~bits + 1u : bits | 0x80000000u;
    };
    const bool nan = std::isnan(a) || std::isnan(b);
    const uint32_t x = biased(a), y = biased(b);
    if (!nan && (x > y ? x - y : y - x) <= 4u) return AssertionResult(true);
    return AssertionResult(false, Sides(a_text, b_text, a, b, "=="));
}
inline AssertionResult CmpBool(const char* text, bool value, bool expected) {
    if (value == expected) return AssertionResult(true);
    return AssertionResult(false, std::string("Value of: ") + text + "\n  Actual: " + (value ? "true" : "false") +
                                      "\nExpected: " + (expected ? "true" : "false"));
}

inline bool MatchesPattern(const char* pattern, const char* text) {
    if (*pattern == '\0') return *text == '\0';
    if (*pattern == '*') return MatchesPattern(pattern + 1, text) || (*text != '\0' && MatchesPattern(pattern, text + 1));
    if (*pattern == '?') return *text != '\0' && MatchesPattern(pattern + 1, text + 1);
    return *pattern == *text && MatchesPattern(pattern + 1, text + 1);
}
inline bool MatchesAny(const std::string& patterns, const std::string& name) {
    size_t start = 0;
    while (start <= patterns.size()) {
        size_t end = patterns.find(':', start);
        if (end == std::string::npos) end = patterns.size();
        const std::string one = patterns.substr(start, end - start);
        if (!one.empty() && MatchesPattern(one.c_str(), name.c_str())) return true;
        start = end + 1;
    }
    return false;
}

inline int RunAllTests(int argc, char** argv) {
    std::string positive = "*", negative;
    bool list_only = false;
    for (int i = 1; i < argc; ++i) {
        const std::string arg = argv[i];
        if (arg.rfind("--gtest_filter=", 0) == 0) {
            const std::string filter = arg.substr(15);
            const size_t dash = filter.find('-');
            positive = dash == std::string::npos ? filter : filter.substr(0, dash);
            negative = dash == std::string::npos ? std::string() : filter.substr(dash + 1);
            if (positive.empty()) positive = "*";
        } else if (arg == "--gtest_list_tests") {
            list_only = true;
        }
    }
    int passed = 0, failed = 0, skipped = 0;
    std::vector<std::string> failed_names;
    for (const Case& c : Cases()) {
        if (!MatchesAny(positive, c.name) || (!negative.empty() && MatchesAny(negative, c.name))) continue;
        if (list_only) {
            std::printf("%s\n", c.name.c_str());
            continue;
        }
        State() = CaseState{};
        std::printf("[ RUN      ] %s\n", c.name.c_str());
        std::fflush(stdout);
        c.body();
        if (State().failures > 0) {
            ++failed;
            failed_names.push_back(c.name);
            std::printf("[  FAILED  ] %s\n", c.name.c_str());
        } else if (State().skipped) {
            ++skipped;
            std::printf("[  SKIPPED ] %s%s%s\n", c.name.c_str(), State().skip_text.empty() ? "" : ": ", State().skip_text.c_str());
        } else {
            ++passed;
            std::printf("[       OK ] %s\n", c.name.c_str());
        }
        std::fflush(stdout);
    }
    if (list_only) return 0;
    std::printf("[==========] %d tests ran.\n[  PASSED  ] %d tests.\n", passed + failed + skipped, passed);
    if (skipped > 0) std::printf("[  SKIPPED ] %d tests.\n", skipped);
    if (failed > 0) {
        std::printf("[  FAILED  ] %d tests, listed below:\n", failed);
        for (const std::string& name : failed_names) std::printf("[  FAILED  ] %s\n", name.c_str());
    }
    std::printf("SUMMARY passed=%d failed=%d skipped=%d\n", passed, failed, skipped);
    return failed == 0 ? 0 : 1;
}

}  // namespace internal

inline void InitGoogleTest(int*, char**) {}

}  // namespace testing

inline int RUN_ALL_TESTS() { return ::testing::internal::RunAllTests(0, nullptr); }

#define GTEST_SHIM_NAME_(suite, name) suite##_##name##_Test

#define TEST(suite, name)                                                                                      \
    static void GTEST_SHIM_NAME_(suite, name)();                                                                \
    static ::testing::internal::Registrar suite##_##name##_registrar(#suite, #name, GTEST_SHIM_NAME_(suite, name)); \
    static void GTEST_SHIM_NAME_(suite, name)()

// The `switch (0) case 0: default:` prefix makes the if/else below a single statement that tolerates a dangling else.
#define GTEST_SHIM_NONFATAL_(result_expr)                                        \
    switch (0)                                                                   \
    case 0:                                                                      \
    default:                                                                     \
        if (const ::testing::AssertionResult gtest_shim_r = (result_expr)) {     \
        } else                                                                   \
            ::testing::internal::Reporter(__FILE__, __LINE__, false, gtest_shim_r.text()) = ::testing::Message()

#define GTEST_SHIM_FATAL_(result_expr)                                           \
    switch (0)                                                                   \
    case 0:                                                                      \
    default:                                                                     \
        if (const ::testing::AssertionResult gtest_shim_r = (result_expr)) {     \
        } else                                                                   \
            return ::testing::internal::Reporter(__FILE__, __LINE__, true, gtest_shim_r.text()) = ::testing::Message()

#define EXPECT_TRUE(x) GTEST_SHIM_NONFATAL_(::testing::internal::CmpBool(#x, static_cast<bool>(x), true))
#define EXPECT_FALSE(x) GTEST_SHIM_NONFATAL_(::testing::internal::CmpBool(#x, static_cast<bool>(x), false))
#define ASSERT_TRUE(x) GTEST_SHIM_FATAL_(::testing::internal::CmpBool(#x, static_cast<bool>(x), true))
#define ASSERT_FALSE(x) GTEST_SHIM_FATAL_(::testing::internal::CmpBool(#x, static_cast<bool>(x), false))

#define EXPECT_EQ(a, b) GTEST_SHIM_NONFATAL_(::testing::internal::CmpEQ(#a, #b, (a), (b)))
#define EXPECT_NE(a, b) GTEST_SHIM_NONFATAL_(::testing::internal::CmpNE(#a, #b, (a), (b)))
#define EXPECT_LT(a, b) GTEST_SHIM_NONFATAL_(::testing::internal::CmpLT(#a, #b, (a), (b)))
#define EXPECT_LE(a, b) GTEST_SHIM_NONFATAL_(::testing::internal::CmpLE(#a, #b, (a), (b)))
#define EXPECT_GT(a, b) GTEST_SHIM_NONFATAL_(::testing::internal::CmpGT(#a, #b, (a), (b)))
#define EXPECT_GE(a, b) GTEST_SHIM_NONFATAL_(::testing::internal::CmpGE(#a, #b, (a), (b)))
#define ASSERT_EQ(a, b) GTEST_SHIM_FATAL_(::testing::internal::CmpEQ(#a, #b, (a), (b)))
#define ASSERT_NE(a, b) GTEST_SHIM_FATAL_(::testing::internal::CmpNE(#a, #b, (a), (b)))
#define ASSERT_LT(a, b) GTEST_SHIM_FATAL_(::testing::internal::CmpLT(#a, #b, (a), (b)))
#define ASSERT_LE(a, b) GTEST_SHIM_FATAL_(::testing::internal::CmpLE(#a, #b, (a), (b)))
#define ASSERT_GT(a, b) GTEST_SHIM_FATAL_(::testing::internal::CmpGT(#a, #b, (a), (b)))
#define ASSERT_GE(a, b) GTEST_SHIM_FATAL_(::testing::internal::CmpGE(#a, #b, (a), (b)))

#define EXPECT_STREQ(a, b) GTEST_SHIM_NONFATAL_(::testing::internal::CmpStrEq(#a, #b, (a), (b)))
#define ASSERT_STREQ(a, b) GTEST_SHIM_FATAL_(::testing::internal::CmpStrEq(#a, #b, (a), (b)))
#define EXPECT_NEAR(a, b, tol) GTEST_SHIM_NONFATAL_(::testing::internal::CmpNear(#a, #b, (a), (b), (tol)))
#define ASSERT_NEAR(a, b, tol) GTEST_SHIM_FATAL_(::testing::internal::CmpNear(#a, #b, (a), (b), (tol)))
#define EXPECT_FLOAT_EQ(a, b) GTEST_SHIM_NONFATAL_(::testing::internal::CmpFloatEq(#a, #b, (a), (b)))
#define ASSERT_FLOAT_EQ(a, b) GTEST_SHIM_FATAL_(::testing::internal::CmpFloatEq(#a, #b, (a), (b)))

#define ADD_FAILURE() ::testing::internal::Reporter(__FILE__, __LINE__, false, "Failed") = ::testing::Message()
#define FAIL() return ::testing::internal::Reporter(__FILE__, __LINE__, true, "Failed") = ::testing::Message()
#define SUCCEED() ::testing::Message()
#define GTEST_SKIP() return ::testing::internal::Skipper() = ::testing::Message()

#if defined(GTEST_SHIM_MAIN)
int main(int argc, char** argv) { return ::testing::internal::RunAllTests(argc, argv); }
#endif
