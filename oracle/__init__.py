"""CPU oracle of the KV movement path: test infrastructure, never imported by the product."""
