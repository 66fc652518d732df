module gmoracle

go 1.20
