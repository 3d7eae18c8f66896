"""What one step runs: for each request its next tokens and the places whose logits are wanted."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, List, Optional, Sequence

import torch


@dataclass
class StepEntry:
    rid: Hashable
    tokens: Sequence[int]                 # the request's next tokens (a prompt portion, or one decoded token)
    want: Sequence[int] = ()              # indices into `tokens` whose logits are returned


@dataclass
class StepContext:
    """The batch as the parts see it.  All tensors are int32 on the device.

    Rows of the step are the entries' tokens back to back.  positions[t] is the row's position in
    its request, req_of_token[t] the request's index within this step, q_start the prefix sums of
    the entries' lengths, pos_start the first position of each entry, slot_ids each request's
    state slot, block_tables[g] the page table [R, blocks] of cache group g, logit_rows the rows
    whose logits are wanted."""
    T: int
    R: int
    token_ids: torch.Tensor
    positions: torch.Tensor
    req_of_token: torch.Tensor
    q_start: torch.Tensor
    pos_start: torch.Tensor
    slot_ids: torch.Tensor
    block_tables: List[torch.Tensor]
    logit_rows: torch.Tensor
    n_logit_rows: int
    # host copies, for parts that plan their launches
    q_lens: List[int] = field(default_factory=list)
    pos_starts: List[int] = field(default_factory=list)
    slots: List[int] = field(default_factory=list)
    max_context: int = 0                  # largest position + 1 in the step
    max_q_len: int = 0
    plans: dict = field(default_factory=dict)     # per-step launch plans that parts share across layers (keyed by the part)
    made: set = field(default_factory=set)        # keys of plans whose device-side part has been launched in this pass over the
                                                  # layers: the runner empties it before it records the step, so that a kernel
                                                  # that fills a plan from the step's positions is part of the recording
    fed: Optional[torch.Tensor] = None            # int32 ids the step before sampled: a token id -(i + 1) stands for fed[i]
    position: int = 0                             # the executed position (index into the model's order) whose block is running

    def query_tiles(self, tokens_per_tile: int, at_most: Optional[int] = None):
        """Tiles of at most `tokens_per_tile` consecutive tokens of one request, as device arrays
        (first row, token count) and their number; made once per step and size.  at_most: only
        the requests that bring at most that many tokens to the step."""
        key = ("query_tiles", tokens_per_tile, at_most)
        if key not in self.plans:
            first, count, at = [], [], 0
            for n in self.q_lens:
                if at_most is None or n <= at_most:
                    for i in range(0, n, tokens_per_tile):
                        first.append(at + i)
                        count.append(min(tokens_per_tile, n - i))
                at += n
            both = torch.tensor([first, count], dtype=torch.int32).reshape(2, -1).to(self.token_ids.device, non_blocking=True)
            self.plans[key] = (both[0], both[1], len(first))
        return self.plans[key]

    def short_requests(self, at_most: int):
        """The requests that bring at most `at_most` tokens to the step: (how many, first row,
        end row, most tokens of one, largest position + 1); rows of other requests may lie between."""
        key = ("short_requests", at_most)
        if key not in self.plans:
            count, lo, hi, most, reach, at = 0, 0, 0, 0, 0, 0
            for r, n in enumerate(self.q_lens):
                if n <= at_most:
                    lo = at if count == 0 else lo
                    count, hi, most = count + 1, at + n, max(most, n)
                    reach = max(reach, (self.pos_starts[r] if r < len(self.pos_starts) else 0) + n)
                at += n
            self.plans[key] = (count, lo, hi, most, reach)
        return self.plans[key]

    def query_tile_pairs(self, tokens_per_tile: int, zigzag: bool, more_than: int = 0):
        """The same tiles two by two, both of one request, as device arrays [pairs, 2] (first row,
        token count; a lone tile's partner has no tokens) and their number.  zigzag: a request's
        last tile goes with its first, the one before with the second, ... (under a causal mask
        the late tile's keys include the early tile's, and every pair has the same amount of work);
        else neighbours go together (their key ranges nearly coincide: the choice for a window).
        The pairs come sorted by the number of keys they see, most first.  more_than: only the
        requests that bring more than that many tokens to the step."""
        key = ("query_tile_pairs", tokens_per_tile, zigzag, more_than)
        if key not in self.plans:
            pairs, at = [], 0                            # (keys the pair's later tile sees, first rows, counts)
            for r, n in enumerate(self.q_lens):
                if n <= more_than:
                    at += n
                    continue
                tiles = [(at + i, min(tokens_per_tile, n - i)) for i in range(0, n, tokens_per_tile)]
                k = len(tiles)
                start = self.pos_starts[r] if r < len(self.pos_starts) else 0
                keys = lambda t: start + (t[0] - at) + t[1]
                order = [(k - 1 - j, j) for j in range(k // 2)] if zigzag else [(j + 1, j) for j in range(0, k - 1, 2)]
                for a, b in order:                       # the later tile first: it decides the pair's key range
                    pairs.append((keys(tiles[a]), [tiles[a][0], tiles[b][0]], [tiles[a][1], tiles[b][1]]))
                if k % 2:
                    lone = tiles[k // 2] if zigzag else tiles[k - 1]
                    pairs.append((keys(lone), [lone[0], lone[0]], [lone[1], 0]))
                at += n
            pairs.sort(key=lambda p: -p[0])              # the pairs with the most keys first (stable: ties keep their order)
            first, count = [p[1] for p in pairs], [p[2] for p in pairs]
            both = torch.tensor([first, count], dtype=torch.int32).reshape(2, -1, 2).to(self.token_ids.device, non_blocking=True)
            self.plans[key] = (both[0].contiguous(), both[1].contiguous(), len(first))
        return self.plans[key]
