"""Entry point for corpus preparation that leaves through ``os._exit``.

The pretraining CLI is run with ``--stage prepare``; when it returns, buffered output is flushed
and the interpreter exits immediately, skipping module finalisers -- Arrow / datasets worker
pools have crashed in their finalisers after all output was already durable (the reference
does the same, ops/prepare_data.py:1-33).
"""
from __future__ import annotations

import os
import sys


def main(argv=None) -> None:
    from ..train import pretrain
    code = 0
    try:
        pretrain.main(argv)
    except SystemExit as stop:
        code = stop.code if isinstance(stop.code, int) else (0 if stop.code is None else 1)
    except BaseException:  # noqa: BLE001
        import traceback
        traceback.print_exc()
        code = 1
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(code)


if __name__ == "__main__":
    main()
