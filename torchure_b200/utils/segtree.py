"""Array-backed segment tree answering "smallest marked key >= c" in O(log n).

Used by best-fit-decreasing packing: key s is marked while some open bin has exactly s free
slots (the reference keeps a pointer-based tree of ``Node`` objects, ``torchure/utils.py:45-80``;
this one is a flat bottom-up array).
"""

from __future__ import annotations


class MarkedKeys:
    def __init__(self, n_keys: int):
        size = 1
        while size < n_keys:
            size *= 2
        self.size = size
        self.n_keys = n_keys
        # tree[i] = largest marked key in the subtree, -1 if none
        self.tree = [-1] * (2 * size)

    def set(self, key: int, marked: bool) -> None:
        i = key + self.size
        self.tree[i] = key if marked else -1
        i //= 2
        while i >= 1:
            left, right = self.tree[2 * i], self.tree[2 * i + 1]
            self.tree[i] = left if left > right else right
            i //= 2

    def smallest_at_least(self, c: int) -> int | None:
        """Smallest marked key >= c, or None."""
        if c >= self.n_keys or self.tree[1] < c:
            return None
        i = 1
        while i < self.size:
            # prefer the left child when it still holds a key >= c (its keys are smaller)
            if self.tree[2 * i] >= c:
                i = 2 * i
            else:
                i = 2 * i + 1
        return self.tree[i]
