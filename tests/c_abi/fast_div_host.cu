// Host-only check of the item -> (row slot, tile) division of the streaming kernels:
// fast_div() prepares a multiplier and a shift, and (n * magic) >> (32 + shift) must equal
// n / d for every numerator below 2^31.  Exhaustive over small divisors at the numerators where
// a rounding error would show (multiples of d and their neighbours), plus pseudo-random pairs.
#include <cstdint>
#include <cstdio>

#include "stream.cuh"

static uint32_t quotient(uint32_t n, const cb200::FastDiv& f) {
  if (f.divisor == 1u) return n;
  return static_cast<uint32_t>((static_cast<uint64_t>(n) * f.magic) >> 32) >> f.shift;
}

int main() {
  uint64_t checked = 0, state = 0x9e3779b97f4a7c15ull;
  auto next = [&]() {
    state ^= state << 13; state ^= state >> 7; state ^= state << 17;
    return state;
  };
  auto check = [&](uint32_t n, uint32_t d) {
    const cb200::FastDiv f = cb200::fast_div(d);
    if (quotient(n, f) != n / d) {
      std::printf("fast_div fails: %u / %u gives %u\n", n, d, quotient(n, f));
      return false;
    }
    ++checked;
    return true;
  };
  const uint32_t top = 0x7fffffffu;
  for (uint32_t d = 1; d <= 70000; ++d) {
    const uint32_t around[] = {0u, 1u, d - 1, d, d + 1, 2 * d - 1, 2 * d, top, top - 1, top - d, top / d * d, top / d * d - 1};
    for (uint32_t n : around) {
      if (n <= top && !check(n, d)) return 1;
    }
  }
  for (int i = 0; i < 2000000; ++i) {
    const uint32_t d = static_cast<uint32_t>(next() % top) + 1u;
    const uint32_t n = static_cast<uint32_t>(next() % (static_cast<uint64_t>(top) + 1));
    const uint32_t edge = n / d * d;   // a multiple of d, and the value just below it
    if (!check(n, d) || !check(edge, d) || (edge > 0 && !check(edge - 1, d))) return 1;
  }
  std::printf("fast_div ok: %llu divisions\n", static_cast<unsigned long long>(checked));
  return 0;
}
