"""CPU oracle of the Mooncake EP dispatch/combine path - test infrastructure only."""
