"""Entry points that the reference keeps under ``transformer_nuggets/cute``."""
