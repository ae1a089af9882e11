"""CPU: host-side logic of the peer collectives (slice ownership)."""
import pytest

from flash_attn_v100_b200.comm import slice_bounds


def test_slices_partition_the_vector():
    for world in (1, 2, 4, 8):
        n = 8 * world * 37
        covered = []
        for r in range(world):
            lo, hi = slice_bounds(n, world, r)
            assert (hi - lo) % 8 == 0
            covered += list(range(lo, hi))
        assert covered == list(range(n))
    with pytest.raises(ValueError):
        slice_bounds(100, 8, 0)
