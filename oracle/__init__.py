"""CPU oracle for the MTA forward path: test infrastructure, never on the product path."""
