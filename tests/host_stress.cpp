// Random operations on the native cache manager (csrc/host/page_cache.cpp) with an audit after every one; built
// with AddressSanitizer and UndefinedBehaviorSanitizer by tests/test_host_library_sanitizers.py.
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>
extern "C" {
void* xrh_cache_create(int, const int*, int, int, int, int, int32_t**);
void xrh_cache_destroy(void*);
int xrh_open(void*); int xrh_close(void*, int); long long xrh_length(void*, int);
int xrh_can_reserve(void*, int, long long); int xrh_reserve(void*, int, long long); int xrh_commit(void*, int); int xrh_cancel(void*, int);
int xrh_release_behind_window(void*, int); int xrh_audit(void*, char*, int); int xrh_pages_needed(void*, int, long long, int*);
long long xrh_describe(void*, int, const int*, const int*, const int*, const int*, const int*, int, int, int32_t*, int32_t*, int32_t*, int32_t*, int32_t*, int32_t*, int32_t*, int32_t*, int32_t**);
}
int main() {
    srand(1);
    for (int trial = 0; trial < 200; trial++) {
        int G = 1 + rand() % 2, ps = 1 << (rand() % 5), n_pages = 8 + rand() % 30, mr = 1 + rand() % 5, mp = 12;
        int windows[2] = {-1, 3 + rand() % 20};
        std::vector<std::vector<int32_t>> tabs(G, std::vector<int32_t>((size_t)mr * mp));
        int32_t* tp[2] = {tabs[0].data(), G > 1 ? tabs[1].data() : nullptr};
        void* c = xrh_cache_create(G, windows, n_pages, ps, mr, mp, tp);
        std::vector<int> open;
        char msg[256];
        for (int it = 0; it < 2000; it++) {
            int op = rand() % 10;
            if (op < 2) { int s = xrh_open(c); if (s >= 0) open.push_back(s); }
            else if (op < 8 && !open.empty()) {
                int s = open[rand() % open.size()]; long long n = 1 + rand() % (3 * ps);
                int need[2]; xrh_pages_needed(c, s, n, need);
                if (xrh_can_reserve(c, s, n)) {
                    if (xrh_reserve(c, s, n) != 0) { printf("reserve failed after can_reserve\n"); return 1; }
                    // describe with this one segment (and a filler)
                    std::vector<int> toks((size_t)n, 5); int slot = s, cnt = (int)n, wc = 1, w = (int)n - 1;
                    std::vector<int32_t> a(n + 1), b(n + 1), d(n + 1), rows(2), s0(2), s1(2), s2(2), s3(2);
                    std::vector<std::vector<int32_t>> bt(G, std::vector<int32_t>((size_t)2 * mp));
                    int32_t* btp[2] = {bt[0].data(), G > 1 ? bt[1].data() : nullptr};
                    if (xrh_describe(c, 1, &slot, &cnt, toks.data(), &wc, &w, 1, n_pages, a.data(), b.data(), d.data(), rows.data(), s0.data(), s1.data(), s2.data(), s3.data(), btp) < 0) { printf("describe failed\n"); return 1; }
                    if (rand() % 6 == 0) xrh_cancel(c, s); else xrh_commit(c, s);
                } else if (xrh_reserve(c, s, n) == 0) { printf("reserve succeeded after !can_reserve\n"); return 1; }
            } else if (!open.empty()) {
                size_t k = rand() % open.size(); xrh_close(c, open[k]); open.erase(open.begin() + (long)k);
            }
            if (xrh_audit(c, msg, 256)) { printf("audit: %s\n", msg); return 1; }
        }
        xrh_cache_destroy(c);
    }
    printf("ok\n");
    return 0;
}
