"""Same-GPU comparison arm: the reference project's own final kernel, built unmodified into
baseline/_ref/ (see baseline/Makefile). Used by bench.py and by one GPU cross-check test; never
imported by the b200_attention_b200 package."""
