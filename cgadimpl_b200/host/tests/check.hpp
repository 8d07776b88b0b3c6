// check.hpp -- tiny assertion helpers for the host-layer test programs (plain main() executables,
// like the reference's own tests).
#pragma once
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <functional>
#include <iostream>
#include <string>
#include <vector>

static int g_failures = 0;

#define CHECK(cond)                                                                  \
    do {                                                                             \
        if (!(cond)) {                                                               \
            std::fprintf(stderr, "  CHECK failed: %s  (%s:%d)\n", #cond, __FILE__, __LINE__); \
            ++g_failures;                                                            \
        }                                                                            \
    } while (0)

inline bool run_test(const std::string& name, const std::function<void()>& fn) {
    const int before = g_failures;
    std::printf("Testing: %-44s ", name.c_str());
    std::fflush(stdout);
    try {
        fn();
    } catch (const std::exception& e) {
        std::fprintf(stderr, "  exception: %s\n", e.what());
        ++g_failures;
    }
    const bool ok = g_failures == before;
    std::printf("[%s]\n", ok ? "PASS" : "FAIL");
    return ok;
}

// |a-b| <= atol + rtol*|b| for every element
inline bool all_close(const std::vector<float>& a, const std::vector<float>& b, double rtol, double atol,
                      const char* what = "") {
    if (a.size() != b.size()) {
        std::fprintf(stderr, "  %s: size %zu vs %zu\n", what, a.size(), b.size());
        return false;
    }
    size_t bad = 0, worst = 0;
    double worst_err = 0;
    for (size_t i = 0; i < a.size(); ++i) {
        const double err = std::fabs(double(a[i]) - double(b[i]));
        if (!(err <= atol + rtol * std::fabs(double(b[i])))) {
            ++bad;
            if (err > worst_err || std::isnan(err)) { worst_err = err; worst = i; }
        }
    }
    if (bad)
        std::fprintf(stderr, "  %s: %zu of %zu outside rtol=%g atol=%g; worst at %zu: got %.9g want %.9g\n", what, bad,
                     a.size(), rtol, atol, worst, double(a[worst]), double(b[worst]));
    return bad == 0;
}

inline double frac_equal(const std::vector<float>& a, const std::vector<float>& b) {
    if (a.size() != b.size() || a.empty()) return 0.0;
    size_t eq = 0;
    for (size_t i = 0; i < a.size(); ++i) eq += (a[i] == b[i]) || (std::isnan(a[i]) && std::isnan(b[i]));
    return double(eq) / double(a.size());
}

inline int finish(const char* suite) {
    if (g_failures) std::printf("%s: %d check(s) FAILED\n", suite, g_failures);
    else std::printf("%s: all passed\n", suite);
    return g_failures ? 1 : 0;
}
