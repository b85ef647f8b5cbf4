// Stand-in for the RAFT header of the same name: the two rounding-up divisions the reference uses.
#pragma once
namespace raft {
template <typename S, typename T>
constexpr auto div_rounding_up_unsafe(const S& dividend, const T& divisor) noexcept
{
  return (dividend + divisor - 1) / divisor;
}
template <typename I>
constexpr I div_rounding_up_safe(I dividend, I divisor) noexcept
{
  return dividend / divisor + (dividend % divisor != 0 ? 1 : 0);
}
template <typename I>
constexpr I round_up_unsafe(I v, I m) noexcept
{
  return div_rounding_up_unsafe(v, m) * m;
}
}  // namespace raft
