#!/usr/bin/env python
"""Message passing with per-element ``iris::load`` + ``iris::store`` for the data
(``examples/06_message_passing/message_passing_load_store.py:15-90`` of the reference); same flag protocol as
``message_passing_put.py`` in this directory."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from message_passing_put import main  # noqa: E402

if __name__ == "__main__":
    main(default_variant="load_store")
