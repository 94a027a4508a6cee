"""TEST INFRASTRUCTURE ONLY: CPU restatement of the reference's wavefront 2-D scan.

Nothing in the shipped package ``mamba2d_b200`` imports this package.  It is imported by
``tests/``, by ``__graft_entry__.smoke()`` (as the checker) and by ``bench.py`` for the timed
CPU baseline.
"""
