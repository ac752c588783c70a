// Error text, environment switches and version of libhfrk_b200.so.
#include "host_common.h"

#include <cstdlib>
#include <cstring>
#include <string>

namespace hfrk {

namespace {
thread_local std::string g_last_error;
}

void set_last_error(const char* text) { g_last_error = text ? text : ""; }
void set_last_error_at(const char* text, const char* call) {
    g_last_error = text ? text : "";
    if (call != nullptr) {
        g_last_error += ": ";
        g_last_error.append(call, std::strlen(call) < 160 ? std::strlen(call) : 160);
    }
}

int default_use_pdl() {
    static const int value = [] {
        const char* env = std::getenv("HFRK_PDL");
        return (env != nullptr && std::strcmp(env, "0") == 0) ? 0 : 1;
    }();
    return value;
}

}  // namespace hfrk

extern "C" const char* hfrk_last_error(void) { return hfrk::g_last_error.c_str(); }

extern "C" int hfrk_version(void) { return 100; }
