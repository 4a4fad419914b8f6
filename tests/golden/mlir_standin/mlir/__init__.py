"""Stand-in for the ``mlir`` Python package (test infrastructure, see ``ir.py``)."""
