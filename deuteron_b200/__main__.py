"""`python -m deuteron_b200 KERNEL.ir.json ...`: the compile command (see cli.py)."""
from .cli import main

raise SystemExit(main())
