"""Python mirror of the reference's ``collcache`` package for the extraction path.

``import ugache_b200.collcache.torch as co`` gives the function names of the reference's
``collcache.torch`` (python/collcache/torch/adapter.py:28-55), served by libugache_b200.so.
"""
