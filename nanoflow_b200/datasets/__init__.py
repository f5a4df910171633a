"""Trace generators: fixed-length, real-length (length files) and synthetic log-normal workloads."""
from .traces import (fixed_trace, lognormal_lengths, poisson_arrivals, real_trace, write_trace, read_length_csv,
                     filter_lengths, FIXED_WORKLOADS)
