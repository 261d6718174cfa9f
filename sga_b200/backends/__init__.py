"""Sparse all-reduce transports (the backend plugin axis).

``dense`` is not a class: it is the SGA-off value of ``--sga-backend``; full
steps always use the data-parallel layer's dense synchronisation.
Environment knobs read by the backends:
"""
ENV_ALLOW_RESUME_PIPELINED = "SGA_ALLOW_RESUME_PIPELINED"
ENV_COMM_WARMUP = "SGA_COMM_WARMUP"
