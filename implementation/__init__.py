"""Import names of the reference's ``implementation`` package, served by b200moe."""
