/* Sequential-order WKV-7 recurrence, plain C.  TEST INFRASTRUCTURE (parity oracle).
 *
 * Restates the prototype kernel of the reference (tests/bench_wkv_shared.py:64-97),
 * one "thread" per state row dv, inner loops over dk ascending with a single
 * accumulator each:
 *     sa = sum_dk h[dv][dk] * a[dk]
 *     h[dv][dk] = w[dk] * h[dv][dk] + v[dv] * k[dk] + sa * b[dk]
 *     y[dv] = sum_dk h[dv][dk] * r[dk]
 * r,w,k,v,a,b: [B,T,H,S]; h_in/h_out: [B,H,S,S] (may alias); out: [B,T,H,S].
 * Compile without -ffast-math and with -ffp-contract=off so that the order of
 * roundings is the one written here.
 */
#include <stddef.h>

void wkv7_seq(const float* r, const float* w, const float* k, const float* v, const float* a,
              const float* b, const float* h_in, float* out, float* h_out, int B, int T, int H, int S) {
    for (int bi = 0; bi < B; ++bi)
        for (int hi = 0; hi < H; ++hi)
            for (int dv = 0; dv < S; ++dv) {
                float row[256];
                const size_t hb = (((size_t)bi * H + hi) * S + dv) * S;
                for (int dk = 0; dk < S; ++dk) row[dk] = h_in ? h_in[hb + dk] : 0.0f;
                for (int t = 0; t < T; ++t) {
                    const size_t base = (((size_t)bi * T + t) * H + hi) * S;
                    float sa = 0.0f;
                    for (int dk = 0; dk < S; ++dk) sa += row[dk] * a[base + dk];
                    const float vv = v[base + dv];
                    for (int dk = 0; dk < S; ++dk)
                        row[dk] = w[base + dk] * row[dk] + vv * k[base + dk] + sa * b[base + dk];
                    float y = 0.0f;
                    for (int dk = 0; dk < S; ++dk) y += row[dk] * r[base + dk];
                    out[base + dv] = y;
                }
                for (int dk = 0; dk < S; ++dk) h_out[hb + dk] = row[dk];
            }
}
