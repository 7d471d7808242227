"""Import-name compatibility for the reference's ``models`` package."""
