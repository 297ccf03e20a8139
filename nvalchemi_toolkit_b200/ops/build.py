# SPDX-License-Identifier: Apache-2.0
"""``python -m nvalchemi_toolkit_b200.ops.build [--force]`` compiles the sm_100a extension in-tree."""
import sys

from nvalchemi_toolkit_b200.ops._native import build

if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
