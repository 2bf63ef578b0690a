"""CPU oracle package (test infrastructure only; the shipped library never imports it)."""
