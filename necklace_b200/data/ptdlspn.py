"""torch DataLoader whose worker processes are started with ``spawn`` (reference:
necklace/data/ptdlspn.py holds only the imports).  Forked loader workers inherit a CUDA
context they cannot use; spawned ones start clean."""
import torch.utils.data


def spawn_dataloader(dataset, **kwargs):
    if kwargs.get("num_workers", 0) > 0:
        kwargs.setdefault("multiprocessing_context", "spawn")
        kwargs.setdefault("persistent_workers", True)
    return torch.utils.data.DataLoader(dataset, **kwargs)
