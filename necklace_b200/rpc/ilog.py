"""Integer-channel debug log (reference: necklace/rpc/ilog.py:4-31).

``debug(i, ...)`` prints only when channel ``i`` is enabled; channels 1..9 are on by
default, trainer services use 500000+, 600000+ and 800000+ and enable them with
``il_add``."""
from __future__ import annotations

import sys
import time

IL = list(range(1, 10))


def il_add(i) -> None:
    if i not in IL:
        IL.append(i)


def il_del(i) -> None:
    if i in IL:
        IL.remove(i)


def debug(i, *args, **kwargs) -> None:
    if i in IL:
        print(f"[{time.strftime('%H:%M:%S')}][{i}]", *args, **kwargs)
        sys.stdout.flush()


def debug_any(ids, *args, **kwargs) -> None:
    """One line if any of the channels ``ids`` is enabled (a message that several
    differently numbered channels of the reference's service flavours would carry)."""
    for i in ids:
        if i in IL:
            print(f"[{time.strftime('%H:%M:%S')}][{i}]", *args, **kwargs)
            sys.stdout.flush()
            return
