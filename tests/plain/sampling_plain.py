"""Plain twin of the sampler's counter-based uniform numbers, written apart from
the product's code: three rounds of the splitmix64 finaliser over (seed, request
id, index of the generated token), the top 24 bits as a fraction."""

M = (1 << 64) - 1


def finalise(x):
    x &= M
    x ^= x >> 30
    x = (x * 0xBF58476D1CE4E5B9) & M
    x ^= x >> 27
    x = (x * 0x94D049BB133111EB) & M
    return x ^ (x >> 31)


def uniform(seed, request_id, index):
    x = finalise(seed + 0x9E3779B97F4A7C15)
    x = finalise(x ^ (request_id * 0xD6E8FEB86659FD93 & M))
    x = finalise(x ^ (index * 0xCA5A826395121157 & M))
    return (x >> 40) / 16777216.0
