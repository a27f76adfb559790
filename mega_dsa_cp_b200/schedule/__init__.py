"""Static task-DAG scheduler: host code generation and the device queue format."""
