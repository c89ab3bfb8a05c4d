"""CPU oracle of the Gemma4 decode arithmetic — test infrastructure, not part of the product."""
