// Minimal stand-in for NTL's RR (arbitrary-precision floating point), enough for the scale bookkeeping of the
// ring-packed matrix-multiply path: the reference keeps every ciphertext's scale as an NTL::RR
// (src/ckks/include/Ciphertext.cuh:14, pcmm/MLWECiphertext.cuh:21) and only ever multiplies, divides, compares,
// prints and converts it (pcmm/PPMM_kernel.cuh:283-284,346).  A long double holds the 2^49-sized scales of this
// path exactly.  With the real NTL installed, leave this directory off the include path.
#ifndef CKKS_LLM_COMPAT_NTL_RR_H
#define CKKS_LLM_COMPAT_NTL_RR_H
#include <iostream>
#include <type_traits>

namespace NTL {

class RR {
public:
    long double v = 0.0L;
    RR() {}
    template <class T, class = typename std::enable_if<std::is_arithmetic<T>::value>::type>
    RR(T x) : v((long double)x) {}
    RR& operator*=(const RR& o) { v *= o.v; return *this; }
    RR& operator/=(const RR& o) { v /= o.v; return *this; }
    RR& operator+=(const RR& o) { v += o.v; return *this; }
    RR& operator-=(const RR& o) { v -= o.v; return *this; }
};
inline RR operator*(RR a, const RR& b) { return a *= b; }
inline RR operator/(RR a, const RR& b) { return a /= b; }
inline RR operator+(RR a, const RR& b) { return a += b; }
inline RR operator-(RR a, const RR& b) { return a -= b; }
inline bool operator<(const RR& a, const RR& b) { return a.v < b.v; }
inline bool operator>(const RR& a, const RR& b) { return a.v > b.v; }
inline bool operator==(const RR& a, const RR& b) { return a.v == b.v; }
inline bool operator!=(const RR& a, const RR& b) { return a.v != b.v; }
inline double to_double(const RR& a) { return (double)a.v; }
inline long to_long(const RR& a) { return (long)a.v; }
inline RR to_RR(double x) { return RR(x); }
inline RR power2_RR(long e) { RR r(1); for (long i = 0; i < e; i++) r.v *= 2; for (long i = 0; i > e; i--) r.v /= 2; return r; }
template <class T> T conv(const RR& a) { return (T)a.v; }
inline std::ostream& operator<<(std::ostream& os, const RR& a) { return os << (double)a.v; }

}  // namespace NTL
#endif
