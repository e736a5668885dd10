"""Prefix cache and the absolute chunk grid (host logic, no GPU): a stand-in state whose 'snapshot' is the token list."""
import numpy as np
import pytest

from pyre_b200.prefix import PrefixCache, grid_pieces


class FakeState:
    """Order-sensitive running hash of the tokens fed so far; a forward over pieces must equal one over the whole."""

    def __init__(self):
        self.tokens = []
        self.calls = []

    def reset(self):
        self.tokens = []

    def forward(self, ids):
        self.calls.append(len(ids))
        self.tokens += list(ids)
        h = 1469598103934665603
        for t in self.tokens:
            h = ((h ^ t) * 1099511628211) % (1 << 64)
        return np.array([h % 1000003, len(self.tokens)], dtype=np.float64)

    def snapshot(self):
        return np.array(self.tokens, dtype=np.uint32).tobytes()

    def restore(self, blob):
        self.tokens = np.frombuffer(blob, dtype=np.uint32).tolist()


def test_grid_pieces_end_on_multiples_of_the_chunk():
    assert grid_pieces(0, 700, 256) == [(0, 256), (256, 512), (512, 700)]
    assert grid_pieces(300, 700, 256) == [(300, 512), (512, 700)]          # a resumed prompt first runs up to the grid
    assert grid_pieces(256, 512, 256) == [(256, 512)]
    assert grid_pieces(0, 5, 256) == [(0, 5)]
    assert grid_pieces(0, 0, 256) == []
    assert grid_pieces(0, 700, 256, cut=300) == [(0, 256), (256, 300), (300, 512), (512, 700)]
    assert grid_pieces(0, 700, 256, cut=256) == [(0, 256), (256, 512), (512, 700)]   # a cut on the grid adds nothing


def test_snapshots_on_the_grid_and_resume_from_the_longest_prefix():
    pc = PrefixCache(chunk=8, cut_at_divergence=True)
    st = FakeState()
    a = list(range(100, 130))                          # 30 tokens: snapshots at 8, 16, 24
    la, sa = pc.prefill(st, a)
    assert sa.source == "new" and sa.pieces == [(0, 8), (8, 16), (16, 24), (24, 30)] and sa.snapshots_taken == 3
    assert [len(s.tokens) for s in pc.snaps] == [8, 16, 24]
    # a different continuation after 20 shared tokens: resumes from the snapshot at 16, cuts at the divergence point 20
    b = a[:20] + [7, 7, 7, 7, 7, 7, 7, 7, 7]
    st.reset(); pc.prev_tokens = ()                    # the live state was lost (another client in between)
    lb, sb = pc.prefill(st, b)
    assert sb.source == "snapshot" and sb.cached_n == 16 and sb.pieces == [(16, 20), (20, 24), (24, 29)]
    fresh = FakeState()
    assert np.array_equal(lb, fresh.forward(b))        # the resumed prefill reaches the state of a prefill from scratch
    assert any(len(s.tokens) == 20 for s in pc.snaps)  # the divergence point was snapshotted too


def test_previous_state_is_continued_when_the_prompt_extends_it():
    pc = PrefixCache(chunk=8)
    st = FakeState()
    a = list(range(10))
    pc.prefill(st, a)
    pc.note_generated([55, 56])
    st.forward([55, 56])                                # the caller generated two tokens
    b = a + [55, 56, 1, 2, 3]
    lb, sb = pc.prefill(st, b)
    assert sb.source == "previous" and sb.cached_n == 12 and sb.pieces == [(12, 15)]
    assert np.array_equal(lb, FakeState().forward(b))
    # a prompt that does not extend the live state starts over (recurrent layers cannot roll back)
    c = a[:5] + [9, 9, 9]
    lc, sc = pc.prefill(st, c)
    assert sc.source in ("new", "snapshot") and np.array_equal(lc, FakeState().forward(c))


def test_snapshot_bytes_are_bounded_oldest_first():
    pc = PrefixCache(chunk=4, cap_bytes=4 * 4 * 5)      # room for about 5 chunk-sized token lists
    st = FakeState()
    pc.prefill(st, list(range(40)))
    assert pc.bytes_held() <= pc.cap_bytes or len(pc.snaps) == 1
    assert len(pc.snaps[-1].tokens) == 36               # the newest survives
    off = PrefixCache(chunk=4, enabled=False)
    _, s = off.prefill(FakeState(), list(range(10)))
    assert s.snapshots_taken == 0 and off.snaps == []


def test_empty_prompt_feeds_the_eos_token():
    pc = PrefixCache(chunk=8)
    st = FakeState()
    _, s = pc.prefill(st, [], eos=2)
    assert st.tokens == [2] and s.prompt_n == 1


def test_without_the_divergence_cut_pieces_stay_on_the_grid():
    pc = PrefixCache(chunk=8)
    st = FakeState()
    a = list(range(100, 130))
    pc.prefill(st, a)
    st.reset(); pc.prev_tokens = ()
    _, sb = pc.prefill(st, a[:20] + [7] * 9)
    assert sb.source == "snapshot" and sb.pieces == [(16, 24), (24, 29)]
