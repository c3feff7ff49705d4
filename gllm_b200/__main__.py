import sys

from gllm_b200.cli import main

sys.exit(main())
