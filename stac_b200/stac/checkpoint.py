"""Stream-state checkpoint and resume for the managers of this package.

The reference keeps all stream state in memory only.  ``save_state`` writes the dictionary of
``manager.state_dict()`` (CPU tensors cut to their used extents, Python counters, a format number)
with ``torch.save``; ``load_state`` restores it into a manager constructed with the same arguments.
A restored stream continues with exactly the bits of the uninterrupted one: token indices, voxel
ids, scores, slot maps, pool contents and retrieved pivots.
"""

import torch


def _sync(manager):
    dev = torch.device(manager.device)
    if dev.type == "cuda":
        torch.cuda.synchronize(dev)


def save_state(manager, path: str) -> None:
    _sync(manager)
    torch.save(manager.state_dict(), path)


def load_state(manager, path: str) -> None:
    """The file holds only tensors, lists, numbers, strings, None and nested dicts, so it is read
    with ``weights_only=True``: a checkpoint from an untrusted source cannot run code on load."""
    manager.load_state_dict(torch.load(path, map_location="cpu", weights_only=True))
    _sync(manager)
