"""Stream-state checkpoint and resume for the managers of this package.

The reference keeps all stream state in memory only.  ``save_state`` writes the dictionary of
``manager.state_dict()`` (CPU tensors cut to their used extents, Python counters, a format number)
with ``torch.save``; ``load_state`` restores it into a manager constructed with the same arguments.
A restored stream continues with exactly the bits of the uninterrupted one: token indices, voxel
ids, scores, slot maps, pool contents and retrieved pivots.
"""

import torch


def save_state(manager, path: str) -> None:
    torch.cuda.synchronize(manager.device)
    torch.save(manager.state_dict(), path)


def load_state(manager, path: str) -> None:
    manager.load_state_dict(torch.load(path, map_location="cpu", weights_only=False))
    torch.cuda.synchronize(manager.device)
