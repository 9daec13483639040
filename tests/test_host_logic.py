"""Host-side logic that needs no GPU: the decode-position guard."""
import pytest

from candy_b200.decoder import PositionGuard


def test_position_guard_refuses_to_run_past_max_ctx():
    g = PositionGuard(4)
    g.set(0)
    g.advance(3)          # positions 0, 1, 2 used; next is 3
    g.need(1)             # position 3 is the last that exists
    g.advance(1)
    with pytest.raises(ValueError, match="past max_ctx 4"):
        g.need(1)         # position 4 would index the cache out of bounds
    with pytest.raises(ValueError):
        g.advance(1)
    g.set(2)
    with pytest.raises(ValueError, match="past max_ctx"):
        g.advance(3)      # a replay of three steps from 2 would run at 2, 3, 4
    g.advance(2)


@pytest.mark.parametrize("pos", [-1, 4, 100])
def test_position_guard_rejects_bad_state(pos):
    g = PositionGuard(4)
    with pytest.raises(ValueError, match="outside"):
        g.set(pos)
