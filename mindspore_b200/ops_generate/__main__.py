import sys

from .gen_ops import main

sys.exit(main())
