"""Run-side utilities: metric key grammar and taxonomy, config migrations, weight addressing."""
