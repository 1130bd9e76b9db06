"""CPU oracle for the GPT-2 forward hot path (test infrastructure, not product code)."""
