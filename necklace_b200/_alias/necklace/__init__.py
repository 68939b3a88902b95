"""Stand-in package named ``necklace``: put this file's parent directory on ``PYTHONPATH``
(``python -m necklace_b200.compat --path`` prints it) and scripts written for the reference
import this framework without any edit, in the main process and in every process it spawns.
Importing it installs the alias finder of ``necklace_b200.compat`` and hands the name over to
the real package."""
import sys

import necklace_b200
import necklace_b200.compat as _compat

_compat.install(force=True)
sys.modules[__name__] = necklace_b200
