"""CPU oracle of the decode hot path: test infrastructure, never part of the
shipped library.  Only tests/, the smoke check and the CPU-baseline legs of the
benchmark import this package."""
