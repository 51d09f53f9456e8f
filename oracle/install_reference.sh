#!/bin/sh
# Test infrastructure, not product code.
#
# Makes an importable, numpy-2 / Cython-3 compatible install of the read-only
# reference checkout (IDSIA/brainstorm 0.5) under baseline/_ref/ (git-ignored).
# The reference tree itself is never modified and none of its sources enter the
# history of this repository: the copy is produced from the checkout by this
# recipe every time.
#
# The install is used (1) to validate oracle/numpy_oracle.py against the real
# NumpyHandler and to generate tests/golden/*.npz (tests/golden/make_golden.py),
# and (2) as the *caller* side of the drop-in boundary: the unchanged layers,
# BufferManager, Network, Trainer and steppers that drive B200Handler through
# Network.set_handler (brainstorm/structure/network.py:359).
#
# usage: oracle/install_reference.sh [reference checkout] [target dir]
set -e
HERE=$(cd "$(dirname "$0")/.." && pwd)
REF=${1:-${B200_REFERENCE_SRC:-$HERE/../reference}}
DST=${2:-$HERE/baseline/_ref}
TMP=$(mktemp -d /tmp/bsref.XXXXXX)

cp -r "$REF/brainstorm" "$REF/setup.py" "$REF/README.md" "$REF/HISTORY.rst" "$TMP"/
chmod -R u+w "$TMP"
cd "$TMP"

# numpy >= 1.24 removed the np.Inf / np.bool / np.int / np.float aliases.
sed -i 's/np\.Inf/np.inf/g' brainstorm/training/schedules.py
sed -i 's/dtype=np\.bool)/dtype=bool)/g; s/dtype=np\.int)/dtype=int)/g' brainstorm/data_iterators.py
sed -i 's/dtype=np\.float)/dtype=float)/' brainstorm/initializers.py
sed -i 's/astype(np\.float)/astype(float)/' brainstorm/scorers.py
sed -i 's/astype(np\.int)/astype(int)/' brainstorm/tools.py
# Cython 3 no longer accepts the np.int_t memoryview alias.
sed -i 's/np\.int_t\[:\]/np.int64_t[:]/g' brainstorm/handlers/_cpuop.pyx
# setuptools >= 72 has no setuptools.command.test.
sed -i 's/^from setuptools.command.test import test as TestCommand/TestCommand = object/' setup.py

python3 setup.py build_ext --inplace > "$TMP/build.log" 2>&1 || { tail -30 "$TMP/build.log"; exit 1; }

rm -rf "$DST"
mkdir -p "$DST"
cp -r "$TMP/brainstorm" "$DST/brainstorm"
# h5py is not installed here and is imported at module top by
# structure/network.py, hooks.py and tools.py; `mock` is imported by one test.
mkdir -p "$DST/h5py" "$DST/mock"
printf 'class File(object):\n    def __init__(self, *a, **k):\n        raise ImportError("h5py is not installed (stub)")\n' > "$DST/h5py/__init__.py"
printf 'from unittest.mock import *  # noqa\n' > "$DST/mock/__init__.py"
find "$DST" -name '*.c' -size +100k -delete
rm -rf "$TMP"
echo "reference installed at $DST"
