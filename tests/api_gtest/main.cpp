// Entry point of the binary that runs the reference's API tests against this
// library (the reference's own main registers a harness environment that needs
// the vendor runtime; the tests themselves do not).
#include "gtest/gtest.h"

int main(int argc, char *argv[]) {
  testing::InitGoogleTest(&argc, argv);
  return RUN_ALL_TESTS();
}
