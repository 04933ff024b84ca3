"""Mirror of the reference's `elasticmm.engine` package for the KV movement path."""
