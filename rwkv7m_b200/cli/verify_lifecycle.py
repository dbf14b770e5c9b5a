"""``rwkv7m-verify-lifecycle``: ``create`` in one process, ``restore`` in another
(reference: src/rwkv7m/cli/verify_nnx_lifecycle.py)."""

from __future__ import annotations

import argparse
import json
import sys

from ..parallel.lifecycle import create_lifecycle_checkpoint, restore_lifecycle_checkpoint


def main(argv=None):
    p = argparse.ArgumentParser(description="Probe the create/save/restore lifecycle of a train state.")
    p.add_argument("mode", choices=["create", "restore"])
    p.add_argument("--directory", required=True)
    p.add_argument("--seed", type=int, default=0)
    args = p.parse_args(argv)
    if args.mode == "create":
        print(json.dumps(create_lifecycle_checkpoint(args.directory, args.seed), indent=2))
        return 0
    result = restore_lifecycle_checkpoint(args.directory)
    print(json.dumps(result, indent=2))
    return 0 if result["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())
