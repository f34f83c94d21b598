"""Offline tools (never imported by the engine): checkpoint quantisers, a multi-rank launcher with
per-GPU health probes, and batch/single-row equality probes.  Counterpart of the reference's
``tools/`` (``quant_disk*.py``, ``launch_occamy_*.sh``, ``probe_*.py``)."""
