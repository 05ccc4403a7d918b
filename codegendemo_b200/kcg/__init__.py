"""Operator API of KCG's matmul path (mirror of Runtime/python/kcg)."""
