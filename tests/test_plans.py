"""Host-side decisions about launch shapes that need no GPU."""

from __future__ import annotations

from edgerag_b200.ops.kernels import context_bound


def test_context_bound_is_a_quarter_of_the_power_of_two_bucket():
    """Steps that share a bound share launch shapes and a captured graph: the bound is the page count
    rounded up to a granule, a quarter of the power-of-two bucket it lies in; it is never below the
    count, less than a granule above it, monotonic, and takes two values per bucket (its upper half)."""
    previous = 0
    for pages in range(1, 3000):
        bound, granule = context_bound(pages)
        bucket = max(4, 1 << (pages - 1).bit_length())
        assert granule == max(1, bucket // 4)
        assert pages <= bound < pages + granule and bound % granule == 0 and bound <= bucket
        assert bound >= previous
        previous = bound
    assert [context_bound(p)[0] for p in (1, 4, 5, 40, 41, 48, 49, 64, 65, 512, 513)] == [1, 4, 6, 48, 48, 48, 64, 64, 96, 512, 768]
    assert {context_bound(p)[0] for p in range(513, 1025)} == {768, 1024}
    assert context_bound(0) == context_bound(1)
