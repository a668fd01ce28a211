// Shared by the compile-side and run-side halves of the C ABI.
#pragma once
#include <exception>
#include <string>
namespace llc {
int setError(int code, const std::string& msg);
int statusFor(const std::exception& e);
}
