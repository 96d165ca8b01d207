"""Developer tooling that ships with the package: an owned-process supervisor with device leasing and port
reservation (the reference's xkit), and the test runner over ``tests/tests.toml`` (its xtest)."""
