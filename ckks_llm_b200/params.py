"""Parameter helpers: NTT-friendly prime chains.

The reference hard-codes its chains per logN (src/ckks/include/Params.cuh:9-174); the
benchmark configurations ask for other sizes, so chains are generated: the `count`
largest primes below 2^bits that are 1 mod 2N.
"""


def _is_prime(n):
    if n < 2:
        return False
    for p in (2, 3, 5, 7, 11, 13, 17, 19, 23, 29, 31, 37):
        if n % p == 0:
            return n == p
    d, r = n - 1, 0
    while d % 2 == 0:
        d //= 2
        r += 1
    for a in (2, 3, 5, 7, 11, 13, 17, 19, 23, 29, 31, 37):
        x = pow(a, d, n)
        if x in (1, n - 1):
            continue
        for _ in range(r - 1):
            x = x * x % n
            if x == n - 1:
                break
        else:
            return False
    return True


def ntt_primes(bits, two_n, count, skip=0):
    """The `count` largest primes p < 2^bits with p = 1 (mod two_n), after skipping `skip`."""
    out = []
    c = (1 << bits) - 1
    c -= (c - 1) % two_n
    while len(out) < count + skip:
        if c < (1 << (bits - 1)):
            raise ValueError("ran out of candidates")
        if _is_prime(c):
            out.append(c)
        c -= two_n
    return out[skip:]


# The reference's own logN=16 chain heads (src/ckks/include/Params.cuh:118-150), used by
# the tie-back tests: ring-pack moduli {q0, q1}, special primes p, auxiliary primes t.
REF_LOGN16_Q = [0x20000018e0001, 0x2000001c00001, 0x2000001ca0001, 0x2000001d20001]
REF_LOGN16_P = [0x2000002600001, 0x20000027e0001, 0x2000002800001, 0x20000029e0001]
REF_LOGN16_T = [0xffffffffffc0001, 0xfffffffff840001, 0xfffffffff6a0001, 0xfffffffff5a0001,
                0xfffffffff2a0001, 0xfffffffff240001, 0xffffffffefe0001, 0xffffffffeca0001]
