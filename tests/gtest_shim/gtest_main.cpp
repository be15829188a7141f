// TEST INFRASTRUCTURE: entry point of the reference's C++ test suite built against tests/gtest_shim.
#include <gtest/gtest.h>
int main(int argc, char** argv) {
    ::testing::InitGoogleTest(&argc, argv);
    return RUN_ALL_TESTS();
}
