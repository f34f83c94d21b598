"""Stable module alias: ``python -m coffin_b200.entrypoints.openai.server`` starts the adapter."""
import sys

from ..cli.openai import main

if __name__ == "__main__":
    sys.exit(main())
