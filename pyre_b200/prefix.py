"""Prompt prefill on the absolute chunk grid with a prefix cache of state snapshots.

Host-side mirror of the reference's request loop (run, src/engine_qn.rs:92-139; Snap, src/model/qwen4exp_gguf.rs:3277-3298):

* a prompt is fed in pieces that end on multiples of `chunk` (256) counted from position 0 -- the first piece of a
  resumed prompt only runs up to the next multiple -- so a prompt that starts from a snapshot is split exactly like a
  prefill of the same tokens from scratch and reaches the same state;
* after every piece that ends on the grid (and is not the end of the prompt) the state is snapshotted, keyed by the
  tokens it covers; a later prompt starts from the longest snapshot it strictly extends, or continues the previous
  request's state when that covers more;
* the snapshots are bounded in bytes, oldest dropped first;
* `cut_at_divergence` adds the reference's extra boundary where a prompt leaves the previous one.  The reference takes
  it only with its split-independent (verify-window) prefill; the batched GPU pass here picks its kernels by piece
  length, so a piece cut off the grid changes the rounding of what follows.  It is therefore off by default: with grid
  boundaries only, a resumed prefill is bit-identical to one from scratch.

The state object needs `forward(ids) -> logits`, `snapshot() -> bytes`, `restore(bytes)` and `reset()`:
`pyre_b200.model.State` (the chunks then run as batched passes on the GPU, pb_forward), or a stand-in in tests.
"""
from __future__ import annotations

from dataclasses import dataclass, field

CHUNK = 256


@dataclass
class Snap:
    tokens: tuple
    blob: bytes

    @property
    def nbytes(self) -> int:
        return len(self.blob)


@dataclass
class PrefillStats:
    prompt_n: int = 0       # tokens fed through the model
    cached_n: int = 0       # tokens covered by the state the prompt started from
    source: str = "new"     # "new" | "previous" | "snapshot"
    pieces: list = field(default_factory=list)   # (start, end) of every forward call
    snapshots_taken: int = 0


def grid_pieces(start: int, end: int, chunk: int = CHUNK, cut: int | None = None):
    """(pos, end) pieces that feed tokens [start, end): each runs up to the next multiple of `chunk`; `cut` adds one
    extra boundary (where this prompt leaves the previous one, src/engine_qn.rs:121-124)."""
    out = []
    pos = start
    while pos < end:
        e = min((pos // chunk + 1) * chunk, end)
        if cut is not None and pos < cut < e:
            e = cut
        out.append((pos, e))
        pos = e
    return out


class PrefixCache:
    def __init__(self, chunk: int = CHUNK, cap_bytes: int = 3072 << 20, enabled: bool = True, cut_at_divergence: bool = False):
        self.chunk, self.cap_bytes, self.enabled, self.cut_at_divergence = chunk, cap_bytes, enabled, cut_at_divergence
        self.snaps: list[Snap] = []
        self.prev_tokens: tuple = ()          # tokens the live state has consumed (the previous request)
        self.last_prompt: tuple = ()

    def bytes_held(self) -> int:
        return sum(s.nbytes for s in self.snaps)

    def _best(self, prompt: tuple):
        """Index and length of the longest snapshot that `prompt` strictly extends."""
        best = None
        for i, s in enumerate(self.snaps):
            n = len(s.tokens)
            if n < len(prompt) and prompt[:n] == s.tokens and (best is None or n > best[1]):
                best = (i, n)
        return best

    def prefill(self, state, prompt, eos: int = 0):
        """Bring `state` to the end of `prompt`; returns (logits of the last position, PrefillStats)."""
        prompt = tuple(int(t) for t in prompt) or (int(eos),)
        st = PrefillStats()
        prev = self.prev_tokens
        # the live state is reused only when the new prompt strictly extends it (recurrent layers cannot roll back)
        ext = len(prev) if 0 < len(prev) < len(prompt) and prompt[:len(prev)] == prev else 0
        best = self._best(prompt) if self.enabled else None
        if ext > 0 and (best is None or best[1] <= ext):
            cached, st.source = ext, "previous"
        elif best is not None:
            snap = self.snaps.pop(best[0])
            state.restore(snap.blob)
            self.snaps.append(snap)               # most recently used last
            cached, st.source = best[1], "snapshot"
        else:
            state.reset()                         # a fresh conversation
            cached, st.source = 0, "new"
        st.cached_n, st.prompt_n = cached, len(prompt) - cached
        # also cut (and snapshot) where this prompt leaves the previous one: the next prompt usually shares that prefix
        lcp = 0
        for a, b in zip(self.last_prompt, prompt):
            if a != b:
                break
            lcp += 1
        cut = lcp if self.enabled and self.cut_at_divergence and cached < lcp < len(prompt) else None
        self.last_prompt = prompt
        logits = None
        for (pos, end) in grid_pieces(cached, len(prompt), self.chunk, cut):
            logits = state.forward(list(prompt[pos:end]))
            st.pieces.append((pos, end))
            on_grid = end % self.chunk == 0 or end == cut
            if self.enabled and on_grid and end < len(prompt) and not any(s.tokens == prompt[:end] for s in self.snaps):
                self.snaps.append(Snap(prompt[:end], state.snapshot()))
                st.snapshots_taken += 1
                while len(self.snaps) > 1 and self.bytes_held() > self.cap_bytes:
                    self.snaps.pop(0)
        self.prev_tokens = prompt
        return logits, st

    def note_generated(self, tokens):
        """Tokens the caller fed to the state after the prompt (generation): the live state now covers them too."""
        self.prev_tokens = self.prev_tokens + tuple(int(t) for t in tokens)
