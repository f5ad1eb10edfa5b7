// Recursive (IIR) filtering for the host runtime: a cascade of second-order sections in direct form I, run over the
// rows of a [rows, n] float64 matrix. A recursion cannot be vectorised along time, so rows are the parallel axis
// (one thread per block of rows); every row's arithmetic is the same serial sequence whatever the thread count.
#include <algorithm>
#include <cstdint>
#include <thread>
#include <vector>

extern "C" {

// sos [sections, 5] = (b0, b1, b2, a1, a2), a0 = 1.  state [rows, sections, 4] = (x1, x2, y1, y2), updated in place.
void sbrt_sos_filter_f64(const double* sos, int32_t sections, const double* x, double* y, double* state, int64_t rows,
                         int64_t n, int32_t threads) {
    auto work = [&](int64_t r0, int64_t r1) {
        std::vector<double> buf((size_t)n);
        for (int64_t r = r0; r < r1; ++r) {
            const double* in = x + r * n;
            double* out = y + r * n;
            for (int32_t s = 0; s < sections; ++s) {
                const double b0 = sos[s * 5], b1 = sos[s * 5 + 1], b2 = sos[s * 5 + 2], a1 = sos[s * 5 + 3],
                             a2 = sos[s * 5 + 4];
                double* st = state + (r * sections + s) * 4;
                double x1 = st[0], x2 = st[1], y1 = st[2], y2 = st[3];
                for (int64_t t = 0; t < n; ++t) {
                    const double xt = in[t];
                    const double yt = b0 * xt + b1 * x1 + b2 * x2 - a1 * y1 - a2 * y2;
                    x2 = x1; x1 = xt; y2 = y1; y1 = yt;
                    buf[(size_t)t] = yt;
                }
                st[0] = x1; st[1] = x2; st[2] = y1; st[3] = y2;
                std::copy(buf.begin(), buf.end(), out);
                in = out;
            }
        }
    };
    int64_t nt = std::max<int64_t>(1, std::min<int64_t>(threads, rows));
    if (nt == 1) { work(0, rows); return; }
    std::vector<std::thread> pool;
    int64_t per = (rows + nt - 1) / nt;
    for (int64_t i = 0; i < nt; ++i) {
        int64_t a = i * per, b = std::min(rows, a + per);
        if (a < b) pool.emplace_back(work, a, b);
    }
    for (auto& t : pool) t.join();
}

}  // extern "C"
