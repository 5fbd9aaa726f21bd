"""CPU oracle of the GLA forward path -- test infrastructure, never imported by gtr_b200."""
