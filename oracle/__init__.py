"""CPU oracle for the state-space hot path.  TEST INFRASTRUCTURE ONLY: imported by
tests/, by the smoke check and by the benchmark's CPU-baseline leg, never by the
shipped package.  PARITY UNPINNED for S4/Mamba outputs (see oracle/oracle_body.inc)."""
