"""CPU oracle for the KLA scan path. Test infrastructure only: see kla_oracle.c."""
