"""Grouped GEMM operators and layout / backend helpers (B200 backend)."""
