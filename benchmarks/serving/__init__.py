"""Single-box serving drivers: load generator, configuration sweep, backend-vs-backend correctness check."""
