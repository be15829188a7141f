// TEST INFRASTRUCTURE: a small stand-in for the googletest API, so that the reference's own C++ test files
// (which include <gtest/gtest.h>; the real library cannot be fetched here) compile and run UNCHANGED against
// the B200 backend.  It provides exactly what those files use: TEST / TEST_F, ::testing::Test with SetUp /
// TearDown, EXPECT_/ASSERT_ {EQ, NE, TRUE, FALSE, FLOAT_EQ, NEAR, THROW}, GTEST_SKIP, `<<` messages, RUN_ALL_TESTS.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstring>
#include <functional>
#include <iostream>
#include <memory>
#include <sstream>
#include <string>
#include <type_traits>
#include <vector>

namespace testing {

class Message {
public:
    template <typename T> Message& operator<<(const T& v) { ss_ << v; return *this; }
    std::string str() const { return ss_.str(); }
private:
    std::ostringstream ss_;
};

struct TestState {
    bool failed = false, skipped = false;
    static TestState& current() { static TestState s; return s; }
};

class Test {
public:
    virtual ~Test() = default;
    virtual void SetUp() {}
    virtual void TearDown() {}
    virtual void TestBody() = 0;
};

struct TestInfo { std::string suite, name; std::function<Test*()> make; };
inline std::vector<TestInfo>& registry() { static std::vector<TestInfo> r; return r; }
struct Registrar { Registrar(const char* s, const char* n, std::function<Test*()> f) { registry().push_back({s, n, std::move(f)}); } };

namespace internal {

template <typename T, typename = void> struct is_streamable : std::false_type {};
template <typename T> struct is_streamable<T, std::void_t<decltype(std::declval<std::ostream&>() << std::declval<const T&>())>> : std::true_type {};

template <typename T> std::string print(const T& v);
template <typename T> std::string print_vec(const std::vector<T>& v) {
    std::string s = "{";
    for (size_t i = 0; i < v.size(); ++i) s += (i ? ", " : "") + print(v[i]);
    return s + "}";
}
template <typename T> struct printer {
    static std::string go(const T& v) {
        if constexpr (std::is_same_v<T, std::nullptr_t>) return "nullptr";
        else if constexpr (std::is_enum_v<T>) return std::to_string((long long)v);
        else if constexpr (is_streamable<T>::value) { std::ostringstream o; o << v; return o.str(); }
        else return "<value>";
    }
};
template <typename T> struct printer<std::vector<T>> { static std::string go(const std::vector<T>& v) { return print_vec(v); } };
template <typename T> std::string print(const T& v) { return printer<T>::go(v); }

class AssertHelper {
public:
    AssertHelper(const char* file, int line, std::string text, bool skip = false) : file_(file), line_(line), text_(std::move(text)), skip_(skip) {}
    void operator=(const Message& m) const {
        if (skip_) { TestState::current().skipped = true; std::cout << "  [ SKIPPED ] " << m.str() << "\n"; return; }
        TestState::current().failed = true;
        std::cout << file_ << ":" << line_ << ": Failure\n" << text_;
        if (!m.str().empty()) std::cout << "\n" << m.str();
        std::cout << "\n";
    }
private:
    const char* file_; int line_; std::string text_; bool skip_;
};

template <typename A, typename B> bool eq(const A& a, const B& b) { return a == b; }

inline bool float_eq(float a, float b) {           // within 4 units in the last place, like googletest
    if (std::isnan(a) || std::isnan(b)) return false;
    if (a == b) return true;
    int32_t ia, ib;
    std::memcpy(&ia, &a, 4); std::memcpy(&ib, &b, 4);
    auto biased = [](int32_t i) -> uint32_t { return i < 0 ? ~(uint32_t)i + 1u : (uint32_t)i | 0x80000000u; };
    uint32_t ua = biased(ia), ub = biased(ib);
    return (ua > ub ? ua - ub : ub - ua) <= 4;
}

template <typename A, typename B>
std::string cmp_text(const char* op, const char* ea, const char* eb, const A& a, const B& b) {
    return std::string("Expected: (") + ea + ") " + op + " (" + eb + "), actual: " + print(a) + " vs " + print(b);
}

}  // namespace internal

inline int RunAllTests() {
    int failed = 0, skipped = 0, passed = 0;
    std::vector<std::string> failures;
    for (auto& t : registry()) {
        TestState::current() = TestState();
        std::cout << "[ RUN      ] " << t.suite << "." << t.name << std::endl;
        try {
            std::unique_ptr<Test> test(t.make());
            test->SetUp();
            if (!TestState::current().skipped && !TestState::current().failed) test->TestBody();
            test->TearDown();
        } catch (const std::exception& e) {
            TestState::current().failed = true;
            std::cout << "unexpected exception: " << e.what() << "\n";
        } catch (...) {
            TestState::current().failed = true;
            std::cout << "unexpected exception\n";
        }
        if (TestState::current().failed) { ++failed; failures.push_back(t.suite + "." + t.name); std::cout << "[  FAILED  ] "; }
        else if (TestState::current().skipped) { ++skipped; std::cout << "[  SKIPPED ] "; }
        else { ++passed; std::cout << "[       OK ] "; }
        std::cout << t.suite << "." << t.name << std::endl;
    }
    std::cout << "[==========] " << registry().size() << " tests ran: " << passed << " passed, " << skipped << " skipped, " << failed << " failed\n";
    for (auto& f : failures) std::cout << "[  FAILED  ] " << f << "\n";
    return failed ? 1 : 0;
}

inline void InitGoogleTest(int*, char**) {}

}  // namespace testing

#define RUN_ALL_TESTS() ::testing::RunAllTests()

#define GTEST_TEST_CLASS_(suite, name) suite##_##name##_Test
#define GTEST_DEFINE_(suite, name, parent)                                                                   \
    class GTEST_TEST_CLASS_(suite, name) : public parent { public: void TestBody() override; };              \
    static ::testing::Registrar gtest_reg_##suite##_##name(#suite, #name, [] { return (::testing::Test*)new GTEST_TEST_CLASS_(suite, name); }); \
    void GTEST_TEST_CLASS_(suite, name)::TestBody()
#define TEST_F(fixture, name) GTEST_DEFINE_(fixture, name, fixture)
#define TEST(suite, name) GTEST_DEFINE_(suite, name, ::testing::Test)

#define GTEST_BLOCKER_ switch (0) case 0: default:
#define GTEST_NONFATAL_(cond, text) GTEST_BLOCKER_ if (cond) ; else ::testing::internal::AssertHelper(__FILE__, __LINE__, text) = ::testing::Message()
#define GTEST_FATAL_(cond, text) GTEST_BLOCKER_ if (cond) ; else return ::testing::internal::AssertHelper(__FILE__, __LINE__, text) = ::testing::Message()

#define EXPECT_EQ(a, b) GTEST_NONFATAL_(::testing::internal::eq((a), (b)), ::testing::internal::cmp_text("==", #a, #b, (a), (b)))
#define EXPECT_NE(a, b) GTEST_NONFATAL_(!::testing::internal::eq((a), (b)), ::testing::internal::cmp_text("!=", #a, #b, (a), (b)))
#define ASSERT_EQ(a, b) GTEST_FATAL_(::testing::internal::eq((a), (b)), ::testing::internal::cmp_text("==", #a, #b, (a), (b)))
#define ASSERT_NE(a, b) GTEST_FATAL_(!::testing::internal::eq((a), (b)), ::testing::internal::cmp_text("!=", #a, #b, (a), (b)))
#define EXPECT_TRUE(c) GTEST_NONFATAL_(static_cast<bool>(c), std::string("Expected true: ") + #c)
#define EXPECT_FALSE(c) GTEST_NONFATAL_(!static_cast<bool>(c), std::string("Expected false: ") + #c)
#define ASSERT_TRUE(c) GTEST_FATAL_(static_cast<bool>(c), std::string("Expected true: ") + #c)
#define ASSERT_FALSE(c) GTEST_FATAL_(!static_cast<bool>(c), std::string("Expected false: ") + #c)
#define EXPECT_FLOAT_EQ(a, b) GTEST_NONFATAL_(::testing::internal::float_eq((float)(a), (float)(b)), ::testing::internal::cmp_text("~=", #a, #b, (float)(a), (float)(b)))
#define EXPECT_NEAR(a, b, tol) GTEST_NONFATAL_(std::fabs((double)(a) - (double)(b)) <= (double)(tol), ::testing::internal::cmp_text("near", #a, #b, (double)(a), (double)(b)))
#define EXPECT_THROW(stmt, type)                                                                             \
    GTEST_BLOCKER_ if ([&] { try { stmt; } catch (const type&) { return true; } catch (...) { return false; } return false; }()) ; \
    else ::testing::internal::AssertHelper(__FILE__, __LINE__, std::string("Expected: ") + #stmt + " throws " + #type) = ::testing::Message()
#define GTEST_SKIP() return ::testing::internal::AssertHelper(__FILE__, __LINE__, "", true) = ::testing::Message()
