import sys

from forgetrain_b200.cli import main

sys.exit(main())
