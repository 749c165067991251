"""Mirror of the reference package layout (custom_helper_op/python)."""
