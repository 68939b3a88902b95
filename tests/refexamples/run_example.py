"""``python run_example.py <script of the reference> <its arguments>``: runs a copy of the script
(and of its sibling modules) whose only change is ``import nkb_ref_boot`` in front."""
import os
import runpy
import shutil
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
script = os.path.abspath(sys.argv[1])
tmp = tempfile.mkdtemp(prefix="nkb_refex_")
for f in os.listdir(os.path.dirname(script)):
    if f.endswith(".py"):
        shutil.copy(os.path.join(os.path.dirname(script), f), tmp)
lines = open(script).read().split("\n")
future = [i for i, l in enumerate(lines) if l.startswith("from __future__")]
lines.insert(future[-1] + 1 if future else 0, "import nkb_ref_boot")
dst = os.path.join(tmp, os.path.basename(script))
with open(dst, "w") as f:
    f.write("\n".join(lines))
sys.path[:0] = [tmp, HERE]
os.environ["PYTHONPATH"] = os.pathsep.join([HERE, os.environ.get("PYTHONPATH", "")])
sys.argv = [dst] + sys.argv[2:]
runpy.run_path(dst, run_name="__main__")
