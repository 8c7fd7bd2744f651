import sys

from rl_kernel_b200.validation.cross_config.runner import main

sys.exit(main())
