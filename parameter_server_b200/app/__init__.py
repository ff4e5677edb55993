"""Applications: the linear methods driven by the reference's configuration format."""
