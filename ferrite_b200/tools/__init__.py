"""Black-box clients that talk to a running server over HTTP with the standard library only (the role of the
reference's `tools/conformance/run.py` and `tools/bench/*.py`)."""
