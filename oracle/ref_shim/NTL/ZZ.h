// Stand-in for <NTL/ZZ.h> and <NTL/RR.h>, used only to COMPILE pieces of the
// reference for the oracle when the real NTL library is absent.  Every operation
// type-checks and returns a dummy: the oracle drives the reference's device kernels
// and integer table builders directly and never executes host code that depends on
// big-number values.
#pragma once
#include <iostream>
#include <vector>
namespace NTL {
class Num {
public:
    double v = 0;
    Num() {}
    template <class T, class = decltype(double(T()))> Num(const T& x) : v(double(x)) {}
    static void SetPrecision(long) {}
    static void SetOutputPrecision(long) {}
    Num& operator+=(const Num&) { return *this; }
    Num& operator-=(const Num&) { return *this; }
    Num& operator*=(const Num&) { return *this; }
    Num& operator/=(const Num&) { return *this; }
    Num& operator%=(const Num&) { return *this; }
    Num& operator<<=(long) { return *this; }
    Num& operator>>=(long) { return *this; }
    Num operator-() const { return *this; }
    operator unsigned long long() const { return 0; }
    Num& operator++() { return *this; }
    Num& operator--() { return *this; }
};
typedef Num ZZ;
typedef Num RR;
#define NTL_SHIM_BINOP(op)                                                        \
    inline Num operator op(const Num& a, const Num&) { return a; }                \
    template <class T, class = decltype(double(T()))>                             \
    inline Num operator op(const Num& a, const T&) { return a; }                  \
    template <class T, class = decltype(double(T()))>                             \
    inline Num operator op(const T&, const Num& b) { return b; }
NTL_SHIM_BINOP(+)
NTL_SHIM_BINOP(-)
NTL_SHIM_BINOP(*)
NTL_SHIM_BINOP(/)
NTL_SHIM_BINOP(%)
#undef NTL_SHIM_BINOP
inline Num operator<<(const Num& a, long) { return a; }
inline Num operator>>(const Num& a, long) { return a; }
#define NTL_SHIM_CMP(op)                                                          \
    inline bool operator op(const Num& a, const Num& b) { return a.v op b.v; }    \
    template <class T, class = decltype(double(T()))>                             \
    inline bool operator op(const Num& a, const T& b) { return a.v op double(b); } \
    template <class T, class = decltype(double(T()))>                             \
    inline bool operator op(const T& a, const Num& b) { return double(a) op b.v; }
NTL_SHIM_CMP(==)
NTL_SHIM_CMP(!=)
NTL_SHIM_CMP(<)
NTL_SHIM_CMP(>)
NTL_SHIM_CMP(<=)
NTL_SHIM_CMP(>=)
#undef NTL_SHIM_CMP
inline std::ostream& operator<<(std::ostream& o, const Num&) { return o; }
template <class T> inline Num to_ZZ(const T&) { return Num(); }
template <class T> inline Num to_RR(const T&) { return Num(); }
inline long to_long(const Num&) { return 0; }
inline unsigned long to_ulong(const Num&) { return 0; }
inline int to_int(const Num&) { return 0; }
inline double to_double(const Num&) { return 0; }
template <class T, class S> inline T conv(const S&) { return T(); }
template <class T, class S> inline void conv(T&, const S&) {}
inline Num power(const Num& a, long) { return a; }
inline Num power2_RR(long) { return Num(); }
inline Num pow(const Num& a, const Num&) { return a; }
inline Num sqrt(const Num& a) { return a; }
inline Num abs(const Num& a) { return a; }
inline Num log(const Num& a) { return a; }
inline Num exp(const Num& a) { return a; }
inline Num round(const Num& a) { return a; }
inline Num floor(const Num& a) { return a; }
inline Num ceil(const Num& a) { return a; }
inline Num RoundToZZ(const Num& a) { return a; }
inline Num TruncToZZ(const Num& a) { return a; }
inline Num FloorToZZ(const Num& a) { return a; }
inline Num InvMod(const Num& a, const Num&) { return a; }
inline Num MulMod(const Num& a, const Num&, const Num&) { return a; }
inline Num PowerMod(const Num& a, const Num&, const Num&) { return a; }
inline long NumBits(const Num&) { return 0; }
inline long bit(const Num&, long) { return 0; }
inline void RandomBits(Num&, long) {}
inline Num RandomBits_ZZ(long) { return Num(); }
inline void rem(Num&, const Num&, const Num&) {}
inline void mul(Num&, const Num&, const Num&) {}
inline void add(Num&, const Num&, const Num&) {}
inline void sub(Num&, const Num&, const Num&) {}
inline void div(Num&, const Num&, const Num&) {}
inline void LeftShift(Num&, const Num&, long) {}
inline void RightShift(Num&, const Num&, long) {}
inline void BytesFromZZ(unsigned char*, const Num&, long) {}
inline void ZZFromBytes(Num&, const unsigned char*, long) {}
inline Num ZZFromBytes(const unsigned char*, long) { return Num(); }
}  // namespace NTL
