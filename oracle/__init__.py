"""CPU oracle for the sparse-MLA hot path.  Test infrastructure, not product:
only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
import it."""
