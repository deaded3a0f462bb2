/* TEST INFRASTRUCTURE -- the checker, never the thing shipped or measured.
 *
 * Direct O(N^2) evaluation of the transform the reference computes: forward,
 * unnormalised, X[k] = sum_n x[n] * exp(-2*pi*i*n*k/N)  (sign and scaling fixed by the
 * twiddle table of include/utils/initializeData.h:31-37 and by the cuFFT call the
 * reference verifies against, include/cufft/cufft.h:23, CUFFT_FORWARD).
 * Accumulates in long double with an exactly reduced phase (n*k mod N), so it is
 * independent of every FFT factorisation, including numpy's.
 */
#include <math.h>
#include <stddef.h>

static const long double TWO_PI = 6.283185307179586476925286766559005768L;

/* in/out: batch x n interleaved (re, im) doubles. */
void dft_oracle(const double* in, double* out, long long n, long long batch) {
    for (long long b = 0; b < batch; ++b) {
        const double* x = in + 2 * b * n;
        double* y = out + 2 * b * n;
        for (long long k = 0; k < n; ++k) {
            long double sr = 0.0L, si = 0.0L;
            for (long long j = 0; j < n; ++j) {
                const long long ph = (j * k) % n;
                const long double ang = -TWO_PI * (long double)ph / (long double)n;
                const long double c = cosl(ang), s = sinl(ang);
                sr += (long double)x[2 * j] * c - (long double)x[2 * j + 1] * s;
                si += (long double)x[2 * j] * s + (long double)x[2 * j + 1] * c;
            }
            y[2 * k] = (double)sr;
            y[2 * k + 1] = (double)si;
        }
    }
}

/* A few output bins of one long signal (n up to 2^31): used where a full CPU FFT of
 * the signal would not fit in time or memory. */
void dft_oracle_bins(const double* in, long long n, const long long* bins, int nbins, double* out) {
    for (int q = 0; q < nbins; ++q) {
        const long long k = bins[q];
        long double sr = 0.0L, si = 0.0L;
        for (long long j = 0; j < n; ++j) {
            const long long ph = (long long)(((unsigned __int128)j * (unsigned __int128)k) % (unsigned __int128)n);
            const long double ang = -TWO_PI * (long double)ph / (long double)n;
            const long double c = cosl(ang), s = sinl(ang);
            sr += (long double)in[2 * j] * c - (long double)in[2 * j + 1] * s;
            si += (long double)in[2 * j] * s + (long double)in[2 * j + 1] * c;
        }
        out[2 * q] = (double)sr;
        out[2 * q + 1] = (double)si;
    }
}
