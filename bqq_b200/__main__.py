"""`python -m bqq_b200 <script.py> [args...]`: run a script of the reference project (for example
its lm/build_bqq_model.py or lm/benchmark_inference.py) with this package installed as
`bqq_modules` / `bqq_cuda_ext`, without editing the script.  The scripts put their own `src/`
directory on sys.path and then `from bqq_modules import ...`; an entry in sys.modules wins over
the path, which is all install() does."""
import os
import runpy
import sys

import bqq_b200


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit('usage: python -m bqq_b200 <script.py> [args...]')
    script = sys.argv[1]
    bqq_b200.install()
    sys.argv = sys.argv[1:]
    sys.path.insert(0, os.path.dirname(os.path.abspath(script)))
    runpy.run_path(script, run_name='__main__')


if __name__ == '__main__':
    main()
