"""ThreadBlockGroup: several thread blocks that split one operation between them."""
from __future__ import annotations

from typing import Dict, List


class ThreadBlockGroup:
    def __init__(self, tb_list: List[int]):
        self.tb_list: List[int] = list(tb_list)
        self._position: Dict[int, int] = {}
        for i, tb in enumerate(self.tb_list):
            if tb in self._position:
                raise ValueError(f"Duplicate thread block found at index {i}: {tb}")
            self._position[tb] = i

    def get_internal_id(self, tb: int) -> int:
        if tb not in self._position:
            raise ValueError(f"Thread block {tb} not found in thread block group")
        return self._position[tb]

    def numtb(self) -> int:
        return len(self.tb_list)
