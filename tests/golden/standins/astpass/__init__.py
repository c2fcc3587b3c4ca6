"""Stand-in for the third-party ``astpass`` package (not installed in this image), used ONLY
by tests/golden/make_golden.py.  Each pass is written from how the reference calls it."""
