"""TEST INFRASTRUCTURE: CPU oracle of the GEMM path. Imported only by tests/, by
``__graft_entry__.smoke()`` and by ``bench.py``'s CPU-baseline / reference arm — never by the
product package ``codegendemo_b200``."""
