// The allocation-free reduction across CUDA contexts on one device.
//
// The entry point's scratch is a static device array of the library, and a device symbol has one
// address per context.  A host program that makes another context current (acro_b200_set_context,
// what acro::setCudaContext calls) must therefore get that context's array, not the address
// looked up earlier.  This program runs the reduction in the primary context, in a second context
// created through the driver API, and in the primary context again, each time on device memory
// of that context, and compares every result with a host sum.
//
// Driver API only (looked up at run time), so the program links against nothing but the library.
// Prints "OK" and returns 0; prints "SKIP: <why>" and returns 0 when a second context cannot be
// created on this machine.
#include "acro_b200.h"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <dlfcn.h>
#include <vector>

typedef int (*fn_init)(unsigned);
typedef int (*fn_device_get)(int *, int);
typedef int (*fn_retain)(void **, int);
typedef int (*fn_release)(int);
typedef int (*fn_ctx_create)(void **, unsigned, int);
typedef int (*fn_ctx_destroy)(void *);
typedef int (*fn_alloc)(unsigned long long *, size_t);
typedef int (*fn_free)(unsigned long long);
typedef int (*fn_h2d)(unsigned long long, const void *, size_t);
typedef int (*fn_d2h)(void *, unsigned long long, size_t);
typedef int (*fn_sync)(void);

static void *driver = nullptr;
template <class F>
static F sym(const char *name)
{
    void *p = dlsym(driver, name);
    if (p == nullptr) { std::printf("FAILED: %s not found in the driver library\n", name); std::exit(1); }
    return reinterpret_cast<F>(p);
}

#define DRV(call)                                                                       \
    do {                                                                                \
        const int rc_ = (call);                                                         \
        if (rc_ != 0) { std::printf("FAILED: %s returned %d\n", #call, rc_); std::exit(1); } \
    } while (0)

struct Problem
{
    int64_t rows;
    int F;
    std::vector<double> a, w, expect, scale;
    Problem(int64_t rows_, int F_, unsigned seed) : rows(rows_), F(F_), a(rows_ * F_), w(rows_), expect(F_, 0.0), scale(F_, 0.0)
    {
        unsigned long long state = seed * 2654435761ull + 12345ull;
        auto next = [&state]() {
            state = state * 6364136223846793005ull + 1442695040888963407ull;
            return static_cast<double>(state >> 11) * (1.0 / 9007199254740992.0);
        };
        for (double &x : a) x = 2.0 * next() - 1.0;
        for (double &x : w) x = 0.5 + next();
        for (int64_t n = 0; n < rows; ++n)
        {
            for (int f = 0; f < F; ++f)
            {
                expect[f] += a[n * F + f] * w[n];
                scale[f] += std::fabs(a[n * F + f]) * w[n];
            }
        }
    }
};

int main()
{
    driver = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
    if (driver == nullptr) { std::printf("FAILED: no CUDA driver library\n"); return 1; }
    fn_init init = sym<fn_init>("cuInit");
    fn_device_get device_get = sym<fn_device_get>("cuDeviceGet");
    fn_retain retain = sym<fn_retain>("cuDevicePrimaryCtxRetain");
    fn_release release = sym<fn_release>("cuDevicePrimaryCtxRelease_v2");
    fn_ctx_create ctx_create = sym<fn_ctx_create>("cuCtxCreate_v2");
    fn_ctx_destroy ctx_destroy = sym<fn_ctx_destroy>("cuCtxDestroy_v2");
    fn_alloc mem_alloc = sym<fn_alloc>("cuMemAlloc_v2");
    fn_free mem_free = sym<fn_free>("cuMemFree_v2");
    fn_h2d h2d = sym<fn_h2d>("cuMemcpyHtoD_v2");
    fn_d2h d2h = sym<fn_d2h>("cuMemcpyDtoH_v2");
    fn_sync ctx_sync = sym<fn_sync>("cuCtxSynchronize");

    DRV(init(0));
    int dev = 0;
    DRV(device_get(&dev, 0));
    void *primary = nullptr;
    DRV(retain(&primary, dev));

    int failures = 0;
    // one run of the entry point in the context that is current, on memory allocated in it
    auto run_here = [&](const Problem &p, const char *where) {
        unsigned long long da = 0, dw = 0, dout = 0;
        DRV(mem_alloc(&da, p.a.size() * sizeof(double)));
        DRV(mem_alloc(&dw, p.w.size() * sizeof(double)));
        DRV(mem_alloc(&dout, p.F * sizeof(double)));
        DRV(h2d(da, p.a.data(), p.a.size() * sizeof(double)));
        DRV(h2d(dw, p.w.data(), p.w.size() * sizeof(double)));
        std::vector<double> got(p.F, -1.0);
        for (int call = 0; call < 2; ++call)      // the second call meets the first one's leftovers in the array
        {
            const int rc = acro_b200_reduce_batch_noalloc(reinterpret_cast<const double *>(da), reinterpret_cast<const double *>(dw),
                                                          reinterpret_cast<double *>(dout), p.rows, p.F, ACRO_B200_OP_ASSIGN, nullptr);
            if (rc != ACRO_B200_OK) { std::printf("FAILED in %s: status %d: %s\n", where, rc, acro_b200_last_error()); std::exit(1); }
            DRV(ctx_sync());
            DRV(d2h(got.data(), dout, p.F * sizeof(double)));
            for (int f = 0; f < p.F; ++f)
            {
                if (!(std::fabs(got[f] - p.expect[f]) <= 1e-12 * p.scale[f]))
                {
                    ++failures;
                    std::printf("FAILED in %s, call %d, entry %d: %.17g against %.17g\n", where, call, f, got[f], p.expect[f]);
                }
            }
        }
        DRV(mem_free(da));
        DRV(mem_free(dw));
        DRV(mem_free(dout));
    };

    const Problem first(100003, 9, 1), second(70001, 32, 2);
    if (acro_b200_set_context(primary) != ACRO_B200_OK) { std::printf("FAILED: %s\n", acro_b200_last_error()); return 1; }
    run_here(first, "the primary context");

    void *other = nullptr;
    const int created = ctx_create(&other, 0, dev);
    if (created != 0)
    {
        std::printf("SKIP: a second context cannot be created on this device (driver status %d)\n", created);
        release(dev);
        return 0;
    }
    if (acro_b200_set_context(other) != ACRO_B200_OK) { std::printf("FAILED: %s\n", acro_b200_last_error()); return 1; }
    run_here(second, "the second context");
    if (acro_b200_set_context(primary) != ACRO_B200_OK) { std::printf("FAILED: %s\n", acro_b200_last_error()); return 1; }
    run_here(first, "the primary context again");
    if (acro_b200_device_status() != ACRO_B200_OK) { std::printf("FAILED: device status: %s\n", acro_b200_last_error()); return 1; }

    DRV(ctx_destroy(other));
    DRV(release(dev));
    if (failures != 0) return 1;
    std::printf("OK\n");
    return 0;
}
