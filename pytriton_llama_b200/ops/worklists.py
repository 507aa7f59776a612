"""Work lists: integer arrays that an operator set wants packed with a step's other integers.

Some kernels do not walk the flat batch but a list made from it on the host (the single-token
rows for the split-key decode attention, tiles of query rows for the prompt attention).  Which
lists there are, how they are cut and what a padded entry must look like is the operator set's
business, because it follows from its kernels' tile shapes; the engine only packs them into the
step's one integer buffer, pads them to the fixed sizes of a captured step and hands the device
views back in ``StepContext.work``.

An operator set that wants lists has
    ``WORK_LISTS``: name -> ``WorkList``  (what exists, for sizing captured steps), and
    ``plan_step(q_lens, starts) -> {name: [int, ...]}``  (a step's lists, host integers).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Union

import torch

PAD_TOKEN_ROW = "token_row"     # padding entries name a token row of the step that belongs to no request


@dataclass(frozen=True)
class WorkList:
    width: int = 1                           # integers per item
    group: int = 1                           # items come in groups of this many (a captured step pads whole groups)
    pad: Union[int, str] = 0                 # what every integer of a padding item is: a number, or PAD_TOKEN_ROW


@dataclass
class StepWork:
    """One list of a step on the device."""
    tensor: torch.Tensor                     # int32 [items * width]
    items: int
    in_order: bool = False                   # width-1 lists only: the items are simply 0..items-1
