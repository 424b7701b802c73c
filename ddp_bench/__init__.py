"""DDP validation bench: eight small models trained under nine execution modes, to check that every
distributed path converges like the single-device run and to compare their wall time
(counterpart of the reference's ddp-bench crate: src/models/mod.rs, src/config.rs, src/harness.rs,
src/analyze.rs, src/report.rs)."""
