// TEST INFRASTRUCTURE ONLY (part of the parity oracle; never used by the product path).
// Stand-in for <glog/logging.h>, which the reference includes only for logging
// (common/helper.h:67,75; dabnn/bitpack.h:25; dabnn/fconv.h:28) and which is an
// empty, un-vendored submodule in the reference checkout.  All log streams are discarded.
#pragma once
#include <iostream>
#include <sstream>
struct DabnnOracleNullStream {
    template <class T> DabnnOracleNullStream& operator<<(const T&) { return *this; }
    DabnnOracleNullStream& operator<<(std::ostream& (*)(std::ostream&)) { return *this; }
};
#define LOG(severity) DabnnOracleNullStream()
#define VLOG(level) DabnnOracleNullStream()
#define CHECK_EQ(a, b) DabnnOracleNullStream()
