"""Imported first by the copy of a reference example script that ``run_example.py`` makes:
the import alias ``necklace`` -> ``necklace_b200``, a synthetic stand-in for the MNIST download
(no network), the CPU in place of ``cuda:<i>`` (the scripts hard-code ``torch.device(gpu)``),
and in-process torch DataLoaders.  Spawned child processes re-import the main script and so
pass through here again."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch  # noqa: E402
import torchvision.datasets as tvd  # noqa: E402

import necklace_b200.compat  # noqa: E402

necklace_b200.compat.install()


class FakeMNIST(torch.utils.data.Dataset):
    def __init__(self, root=None, train=True, download=False, transform=None, **kw):
        n = 256 if train else 64
        g = torch.Generator().manual_seed(0 if train else 1)
        self.x = torch.rand(n, 1, 28, 28, generator=g)
        self.y = torch.randint(0, 10, (n,), generator=g)

    def __len__(self):
        return len(self.x)

    def __getitem__(self, i):
        return self.x[i], int(self.y[i])


tvd.MNIST = FakeMNIST
_real_device = torch.device


class _CpuDevice:
    def __call__(self, x, *a):
        if isinstance(x, int) or (isinstance(x, str) and x.startswith("cuda")):
            return _real_device("cpu")
        return _real_device(x, *a)

    def __instancecheck__(self, o):
        return isinstance(o, _real_device)


if not isinstance(torch.device, _CpuDevice):
    torch.device = _CpuDevice()
torch.cuda.set_device = lambda *a, **k: None
_DL = torch.utils.data.DataLoader
if _DL.__name__ != "_InProcessLoader":
    class _InProcessLoader(_DL):
        def __init__(self, *a, **k):
            k["num_workers"], k["pin_memory"] = 0, False
            super().__init__(*a, **k)
    torch.utils.data.DataLoader = _InProcessLoader
